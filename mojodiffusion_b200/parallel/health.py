"""Rank health and recovery on the host side.

* ``Heartbeat``: every rank bumps a counter in the job's key-value store between steps; before launching the next step
  a rank asks whether all peers have been seen within ``timeout_s``. A missing rank is found on the host, before any
  collective is enqueued, so nothing waits on the device for a peer that is gone.
* ``StepGuard``: wraps one training step: a failure (exception on this rank, a stale peer, a device status word that
  is not OK) marks the step failed in the store so every rank abandons it between steps.
* ``ElasticRunner``: restart policy: fail the step, tear the process group down, reload the last complete backup and
  restart (process exit is the only clean way to give device memory back).

The reference has a single-process trainer with a supervisor that restarts it from the latest step checkpoint, and a
server that treats a closed worker socket as a recoverable event (serenitymojo/training/train_klein_cadence.mojo:64-75,
serenity-server/crates/ipc/src/lib.rs:34-64, serenitymojo/serve/process_isolated_backend.mojo:131-141); this module is
the multi-rank form of the same policy."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional


class DictStore:
    """In-process stand-in for torch.distributed.Store (tests, single process)."""

    def __init__(self):
        self.d: Dict[str, bytes] = {}

    def set(self, k, v):
        self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        return self.d[k]

    def add(self, k, n):
        v = int(self.d.get(k, b"0")) + n
        self.d[k] = str(v).encode()
        return v

    def check(self, keys):
        return all(k in self.d for k in keys)


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], reason: str):
        super().__init__(f"ranks {ranks}: {reason}")
        self.ranks, self.reason = ranks, reason


class Heartbeat:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "hb", clock=time.monotonic):
        self.store, self.rank, self.world, self.timeout, self.prefix, self.clock = store, rank, world, timeout_s, prefix, clock
        self._seen: Dict[int, tuple] = {}

    def beat(self, step: int) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", f"{step}:{self.store.add(f'{self.prefix}/n/{self.rank}', 1)}")

    def _read(self, r: int) -> Optional[str]:
        k = f"{self.prefix}/{r}"
        if not self.store.check([k]):
            return None
        return self.store.get(k).decode()

    def stale_ranks(self) -> List[int]:
        """Ranks whose heartbeat value has not changed for longer than the timeout (or that never wrote one)."""
        now = self.clock()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
                continue
            if now - last[1] > self.timeout:
                out.append(r)
        return out

    def require_all(self) -> None:
        bad = self.stale_ranks()
        if bad:
            raise RankFailure(bad, f"no heartbeat for more than {self.timeout:.1f}s")


class StepGuard:
    """``with StepGuard(...)``: marks the step failed for all ranks if this rank raises; ``check_peers`` is called
    before the next launch."""

    def __init__(self, store, rank: int, world: int, heartbeat: Optional[Heartbeat] = None, prefix: str = "step"):
        self.store, self.rank, self.world, self.hb, self.prefix = store, rank, world, heartbeat, prefix
        self.step = 0

    def failed_flag(self, step: int) -> str:
        return f"{self.prefix}/failed/{step}"

    def check_peers(self, step: int) -> None:
        if self.store.check([self.failed_flag(step)]):
            who = self.store.get(self.failed_flag(step)).decode()
            raise RankFailure([int(who.split(':')[0])], "peer reported failure: " + who.split(':', 1)[1])
        if self.hb is not None:
            self.hb.require_all()

    def run(self, step: int, fn: Callable, status_check: Optional[Callable[[], None]] = None):
        self.check_peers(step)
        try:
            out = fn()
            if status_check is not None:
                status_check()                 # raises if a device wait ran out (status word != OK)
        except RankFailure:
            raise
        except Exception as e:                  # noqa: BLE001 - every failure of the step is reported to the peers
            self.store.set(self.failed_flag(step), f"{self.rank}:{type(e).__name__}: {e}")
            raise
        if self.hb is not None:
            self.hb.beat(step)
        return out


@dataclass
class RestartDecision:
    restart: bool
    from_backup: Optional[str]
    attempt: int
    reason: str


class ElasticRunner:
    """Supervisor policy: run ``launch(resume_path)``; on failure, find the last complete backup and relaunch, at most
    ``max_restarts`` times. ``launch`` returns normally on success and raises on failure."""

    def __init__(self, workspace: str, max_restarts: int = 3, find_backup: Optional[Callable[[str], Optional[str]]] = None):
        from ..training.loop import find_last_backup
        self.workspace, self.max_restarts = workspace, max_restarts
        self.find_backup = find_backup or find_last_backup
        self.history: List[RestartDecision] = []

    def decide(self, attempt: int, error: BaseException) -> RestartDecision:
        if attempt >= self.max_restarts:
            d = RestartDecision(False, None, attempt, f"giving up after {attempt} restarts: {error}")
        else:
            d = RestartDecision(True, self.find_backup(self.workspace), attempt + 1, str(error))
        self.history.append(d)
        return d

    def run(self, launch: Callable[[Optional[str]], None]) -> int:
        attempt, resume = 0, None
        while True:
            try:
                launch(resume)
                return attempt
            except Exception as e:               # noqa: BLE001
                d = self.decide(attempt, e)
                if not d.restart:
                    raise
                attempt, resume = d.attempt, d.from_backup
