"""Config-driven training run: dataset epochs -> step -> cadence actions (sample, save, backup), progress line, board,
resume. File naming, cadence units and resume rules follow the OneTrainer workspace layout:

    <workspace>/save/<prefix><timestamp>-save-<global_step>-<epoch>-<epoch_step>.safetensors
    <workspace>/backup/<timestamp>-backup-<global_step>-<epoch>-<epoch_step>/{meta.json, lora/lora.safetensors,
                                                                          optimizer/optimizer.safetensors}
    <workspace>/samples/<prefix><timestamp>-training-sample-<global_step>-<epoch>-<epoch_step>-<i>.png

Samples run before pending saves of the same step. A LoRA resume requires the optimizer state beside the weights
(serenitymojo/training/onetrainer_resume_contract.mojo:40-160,190-290, onetrainer_train_loop_policy.mojo,
loop.mojo; meta.json carries global_step / epoch / epoch_step / epoch_sample)."""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from ..io.config import TrainConfig
from ..io.safetensors_io import load_safetensors, save_safetensors
from . import features as F
from .board import BoardWriter
from .ema import EMA
from .progress import ProgressDisplay
from .schedule import lr_at


@dataclass
class TrainProgress:
    global_step: int = 0
    epoch: int = 0
    epoch_step: int = 0
    epoch_sample: int = 0

    def filename(self) -> str:
        return f"{self.global_step}-{self.epoch}-{self.epoch_step}"

    def next_step(self, batch_size: int) -> None:
        self.global_step += 1
        self.epoch_step += 1
        self.epoch_sample += batch_size

    def next_epoch(self) -> None:
        self.epoch += 1
        self.epoch_step = 0
        self.epoch_sample = 0


_EXT = {"SAFETENSORS": ".safetensors", "LEGACY_SAFETENSORS": ".safetensors", "CKPT": ".ckpt", "DIFFUSERS": "", "INTERNAL": ""}


def model_file_extension(fmt: str) -> str:
    if fmt not in _EXT:
        raise ValueError(f"unsupported output model format {fmt}")
    return _EXT[fmt]


def step_save_path(workspace: str, prefix: str, timestamp: str, p: TrainProgress, fmt: str = "SAFETENSORS") -> str:
    return os.path.join(workspace, "save", f"{prefix}{timestamp}-save-{p.filename()}{model_file_extension(fmt)}")


def backup_path(workspace: str, timestamp: str, p: TrainProgress) -> str:
    return os.path.join(workspace, "backup", f"{timestamp}-backup-{p.filename()}")


def training_sample_leaf(prefix: str, timestamp: str, p: TrainProgress) -> str:
    return f"{prefix}{timestamp}-training-sample-{p.filename()}"


# ---- cadence: "every N <unit>" with units NEVER | EPOCH | STEP | SECOND | MINUTE | HOUR | ALWAYS ---------------
@dataclass
class TimedAction:
    last_index: int = -1
    started: float = field(default_factory=time.monotonic)


def _unit_position(p: TrainProgress, unit: str, now: float, state: TimedAction) -> float:
    u = unit.upper()
    if u == "EPOCH":
        return p.epoch
    if u == "STEP":
        return p.global_step
    secs = now - state.started
    return {"SECOND": secs, "MINUTE": secs / 60.0, "HOUR": secs / 3600.0}[u]


def single_action_elapsed(state: TimedAction, p: TrainProgress, after: float, unit: str, now: Optional[float] = None) -> bool:
    """True once ``after`` units have passed (used for the skip-first gates)."""
    u = unit.upper()
    if u == "NEVER":
        return False
    if u == "ALWAYS" or after <= 0:
        return True
    return _unit_position(p, u, time.monotonic() if now is None else now, state) >= after


def repeating_action_needed(state: TimedAction, p: TrainProgress, every: float, unit: str, start_at_zero: bool,
                            now: Optional[float] = None) -> bool:
    """True once per interval: at positions k * every (k >= 1, or k >= 0 with ``start_at_zero``). For EPOCH it fires
    on the first step of a due epoch only."""
    u = unit.upper()
    if u == "NEVER" or every <= 0:
        return False
    if u == "ALWAYS":
        return True
    if u == "EPOCH":
        if p.epoch_step != 0:
            return False
        idx = p.epoch // int(every) if p.epoch % int(every) == 0 else -1
    elif u == "STEP":
        idx = p.global_step // int(every) if p.global_step % int(every) == 0 else -1
    else:
        idx = int(_unit_position(p, u, time.monotonic() if now is None else now, state) // every)
    if idx < 0 or idx == state.last_index or (idx == 0 and not start_at_zero):
        return False
    state.last_index = idx
    return True


@dataclass
class ActionDecisions:
    sample: bool
    backup: bool
    save: bool
    sample_before_save: bool = True


class Cadence:
    def __init__(self, cfg: TrainConfig, backup_after: int = 0, backup_after_unit: str = "NEVER"):
        self.cfg = cfg
        self.backup_after, self.backup_unit = backup_after, backup_after_unit
        self.sample_skip, self.sample, self.backup, self.save_skip, self.save = (TimedAction() for _ in range(5))

    def decide(self, p: TrainProgress, now: Optional[float] = None) -> ActionDecisions:
        c = self.cfg
        sample_every = c.sample_after if c.sample_after > 0 else c.sample_every
        s = single_action_elapsed(self.sample_skip, p, c.sample_skip_first, c.sample_after_unit, now) and \
            repeating_action_needed(self.sample, p, sample_every, c.sample_after_unit, True, now)
        b = repeating_action_needed(self.backup, p, self.backup_after, self.backup_unit, False, now)
        v = single_action_elapsed(self.save_skip, p, c.save_skip_first, c.save_every_unit, now) and \
            repeating_action_needed(self.save, p, c.save_every, c.save_every_unit, False, now)
        return ActionDecisions(s, b, v)


# ---- backup / resume -------------------------------------------------------------------------------------------
def write_backup(path: str, progress: TrainProgress, weights: Dict[str, torch.Tensor], optimizer_state: Dict[str, torch.Tensor],
                 model_type: str, training_method: str = "LORA") -> None:
    os.makedirs(os.path.join(path, "lora"), exist_ok=True)
    os.makedirs(os.path.join(path, "optimizer"), exist_ok=True)
    save_safetensors(os.path.join(path, "lora", "lora.safetensors"), weights)
    save_safetensors(os.path.join(path, "optimizer", "optimizer.safetensors"), optimizer_state)
    meta = {"model_type": model_type, "training_method": training_method, "train_progress": {
        "global_step": progress.global_step, "epoch": progress.epoch, "epoch_step": progress.epoch_step,
        "epoch_sample": progress.epoch_sample}}
    tmp = os.path.join(path, "meta.json.tmp")
    with open(tmp, "w") as f:
        json.dump(meta, f)
    os.replace(tmp, os.path.join(path, "meta.json"))     # meta.json last: its presence marks a complete backup


def find_last_backup(workspace: str) -> Optional[str]:
    root = os.path.join(workspace, "backup")
    if not os.path.isdir(root):
        return None
    done = [d for d in sorted(os.listdir(root)) if os.path.isfile(os.path.join(root, d, "meta.json"))]
    return os.path.join(root, done[-1]) if done else None


def read_backup(path: str):
    """Validates the resume manifest and returns (progress, weights, optimizer_state)."""
    mp = os.path.join(path, "meta.json")
    if not os.path.isfile(mp):
        raise FileNotFoundError(f"{path}: meta.json missing; not a complete backup")
    meta = json.load(open(mp))
    tp = meta.get("train_progress", {})
    for k in ("global_step", "epoch", "epoch_step", "epoch_sample"):
        if not isinstance(tp.get(k), int) or tp[k] < 0:
            raise ValueError(f"resume: {k} must be present and non-negative")
    wpath = os.path.join(path, "lora", "lora.safetensors")
    opath = os.path.join(path, "optimizer", "optimizer.safetensors")
    if not os.path.isfile(wpath):
        raise FileNotFoundError("resume: weight state missing")
    if not os.path.isfile(opath):
        raise FileNotFoundError("resume: a LoRA resume requires the optimizer state beside the weights")
    return TrainProgress(tp["global_step"], tp["epoch"], tp["epoch_step"], tp["epoch_sample"]), \
        load_safetensors(wpath), load_safetensors(opath)


# ---- the run -----------------------------------------------------------------------------------------------------
class TrainRun:
    """Glue between a config, a batch loader, a step function and the cadence actions.

    ``step_fn(batch, lr) -> (loss, grad_norm)`` runs one optimizer step; ``named_trainables()`` returns
    {name: tensor} for checkpoints; ``optimizer_state()`` / ``load_optimizer_state(sd)`` expose the moments;
    ``sample_fn(progress, leaf) -> [png paths]`` is optional.

    Multi-rank runs: sampling, backups and saves happen on the main rank only, between steps. ``pre_save_fn`` (optional) is
    called by EVERY rank right before such a branch (gather sharded optimizer state there: collectives inside the
    main-only branch would never be joined); ``barrier_fn`` (optional) is called by every rank right after it, so that the
    other ranks do not enqueue the next step's device-side waits while rank 0 is still writing files; ``agree_fn(bits) ->
    bits`` (optional) replaces this rank's cadence decision by the main rank's (time-based units differ between ranks).
    ``loss_sync_every``: the loss is read back (a host sync) only every that many steps; 1 keeps a full loss history."""

    def __init__(self, cfg: TrainConfig, loader, step_fn: Callable, named_trainables: Callable[[], Dict[str, torch.Tensor]],
                 optimizer_state: Callable[[], Dict[str, torch.Tensor]], load_trainables: Callable, load_optimizer_state: Callable,
                 sample_fn: Optional[Callable] = None, ema: Optional[EMA] = None, board: Optional[BoardWriter] = None,
                 timestamp: Optional[str] = None, prefix: str = "", backup_after: int = 0, backup_after_unit: str = "NEVER",
                 display: bool = True, stream=None, is_main: bool = True, pre_save_fn: Optional[Callable] = None,
                 barrier_fn: Optional[Callable] = None, agree_fn: Optional[Callable] = None, loss_sync_every: int = 1,
                 status_check_fn: Optional[Callable] = None):
        self.cfg, self.loader, self.step_fn = cfg, loader, step_fn
        self.named_trainables, self.optimizer_state = named_trainables, optimizer_state
        self.load_trainables, self.load_optimizer_state = load_trainables, load_optimizer_state
        self.sample_fn, self.ema, self.board = sample_fn, ema, board
        self.timestamp = timestamp or time.strftime("%Y-%m-%d_%H-%M-%S")
        self.prefix = prefix
        self.progress = TrainProgress()
        self.cadence = Cadence(cfg, backup_after, backup_after_unit)
        self.is_main = is_main
        self.display = display and is_main
        self.stream = stream
        self.losses: List[float] = []
        self.saved: List[str] = []
        self.pre_save_fn, self.barrier_fn, self.agree_fn = pre_save_fn, barrier_fn, agree_fn
        self.loss_sync_every = max(1, int(loss_sync_every))
        self.status_check_fn = status_check_fn

    def _decide(self, p: TrainProgress) -> ActionDecisions:
        d = self.cadence.decide(p)
        if self.agree_fn is not None:
            bits = self.agree_fn((int(d.sample) << 2) | (int(d.backup) << 1) | int(d.save))
            d = ActionDecisions(bool(bits & 4), bool(bits & 2), bool(bits & 1))
        return d

    def _act(self, d: ActionDecisions) -> None:
        """Cadence actions of one decision point (every rank calls this; files are written by the main rank)."""
        if not (d.sample or d.backup or d.save):
            return
        if self.status_check_fn is not None:
            self.status_check_fn()                       # a step whose device waits ran out must not be saved
        if (d.backup or d.save) and self.pre_save_fn is not None:
            self.pre_save_fn()
        p = self.progress
        if self.is_main:
            if d.sample and self.sample_fn:
                self.sample_fn(p, training_sample_leaf(self.prefix, self.timestamp, p))
            if d.backup:
                self._backup()
            if d.save:
                self._save()
        if self.barrier_fn is not None:
            self.barrier_fn()

    def resume_if_requested(self) -> bool:
        if not self.cfg.continue_last_backup:
            return False
        last = find_last_backup(self.cfg.workspace_dir)
        if last is None:
            return False
        self.progress, w, o = read_backup(last)
        self.load_trainables(w)
        self.load_optimizer_state(o)
        return True

    def _save(self) -> str:
        path = step_save_path(self.cfg.workspace_dir, self.prefix, self.timestamp, self.progress, self.cfg.output_model_format)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        save_safetensors(path, self.named_trainables(), {"global_step": str(self.progress.global_step)})
        self.saved.append(path)
        return path

    def _backup(self) -> str:
        path = backup_path(self.cfg.workspace_dir, self.timestamp, self.progress)
        write_backup(path, self.progress, self.named_trainables(), self.optimizer_state(), self.cfg.model_type,
                     self.cfg.training_method)
        return path

    def run(self, max_steps: Optional[int] = None) -> TrainProgress:
        cfg = self.cfg
        total = max_steps if max_steps is not None else cfg.total_steps
        spe = max(1, self.loader.steps_per_epoch())
        epochs = (total + spe - 1) // spe
        disp = ProgressDisplay(cfg.model_type, total, epochs, stream=self.stream) if self.display else None
        p = self.progress
        if cfg.sample_at_start and self.sample_fn and self.is_main and p.global_step == 0:
            self.sample_fn(p, training_sample_leaf(self.prefix, self.timestamp, p))
        while p.global_step < total:
            for batch in self.loader.epoch(p.epoch, skip=p.epoch_step):
                if p.global_step >= total:
                    break
                t0 = time.monotonic()
                lr = lr_at(p.global_step, cfg.learning_rate, total, cfg.scheduler_name, cfg.warmup_steps)
                loss, gnorm = self.step_fn(batch, lr)
                p.next_step(cfg.batch_size)
                if self.ema is not None and p.global_step % max(1, cfg.ema_update_step_interval) == 0:
                    self.ema.update(p.global_step)
                if p.global_step % self.loss_sync_every == 0 or p.global_step >= total:
                    loss_f = float(loss)                 # the only host sync of the step
                    self.losses.append(loss_f)
                    if disp:
                        disp.update(p.global_step, p.epoch + 1, loss_f, float(gnorm))
                    if self.board and self.is_main:
                        self.board.log_train_step(p.global_step, loss_f, float(gnorm), lr, time.monotonic() - t0)
                self._act(self._decide(p))
            else:
                p.next_epoch()
                self._act(self._decide(p))               # EPOCH-unit cadences fire here (epoch_step == 0)
                continue
            break
        if disp:
            disp.finish()
        if self.status_check_fn is not None:
            self.status_check_fn()
        if self.pre_save_fn is not None:
            self.pre_save_fn()
        if self.is_main:
            self._backup()
            final = cfg.output_model_destination
            if final:
                dst = final if os.path.isabs(final) else os.path.join(cfg.workspace_dir or ".", final)
                os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
                save_safetensors(dst, self.named_trainables(), {"global_step": str(p.global_step)})
                self.saved.append(dst)
        if self.barrier_fn is not None:
            self.barrier_fn()
        return p
