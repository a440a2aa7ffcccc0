"""Tracing hooks: NVTX ranges around stages, blocks and collectives, and per-rank JSONL metrics with rank-0 aggregation.

Ranges are off by default (``MDB200_NVTX=1`` or ``enable_nvtx(True)`` turns them on) and cost one attribute lookup when
off; with a profiler attached they give the stage / block / collective structure that the reference reconstructs from
kernel grid sizes (BEAT_FLAME_SCOREBOARD_2026-06-10.md:440-465) and from its ``[PROF]`` stage timers
(serenitymojo/training/train_anima_ot.mojo:1078-1121). ``MetricsLog`` is the per-rank JSONL writer; ``aggregate`` folds
the ranks' files into min / max / mean per key for the rank-0 report.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Dict, Iterable, List, Optional

_state = {"on": os.environ.get("MDB200_NVTX", "0") == "1", "depth": 0, "log": None}


def enable_nvtx(on: bool = True) -> None:
    _state["on"] = bool(on)


def nvtx_enabled() -> bool:
    return _state["on"]


def set_range_log(log: Optional[List[str]]) -> None:
    """Tests: record every opened range name into ``log`` (works without a GPU)."""
    _state["log"] = log


@contextlib.contextmanager
def nvtx_range(name: str):
    """``with nvtx_range("block/double/3"):`` — a no-op unless ranges are enabled."""
    if not _state["on"]:
        yield
        return
    log = _state["log"]
    if log is not None:
        log.append(name)
    pushed = False
    try:
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
            pushed = True
    except Exception:
        pushed = False
    try:
        yield
    finally:
        if pushed:
            import torch
            torch.cuda.nvtx.range_pop()


def mark(name: str) -> None:
    if _state["on"]:
        if _state["log"] is not None:
            _state["log"].append("mark:" + name)
        try:
            import torch
            if torch.cuda.is_available():
                torch.cuda.nvtx.mark(name)
        except Exception:
            pass


class MetricsLog:
    """One JSON object per line, one file per rank: ``<dir>/metrics.rank<r>.jsonl``."""

    def __init__(self, directory: str, rank: int = 0):
        os.makedirs(directory, exist_ok=True)
        self.path = os.path.join(directory, f"metrics.rank{rank}.jsonl")
        self.rank = rank
        self._f = open(self.path, "a", buffering=1)

    def log(self, step: int, **values) -> None:
        rec = {"t": round(time.time(), 3), "rank": self.rank, "step": int(step)}
        rec.update({k: (float(v) if hasattr(v, "__float__") else v) for k, v in values.items()})
        self._f.write(json.dumps(rec) + "\n")

    def close(self) -> None:
        self._f.close()


def aggregate(directory: str, keys: Optional[Iterable[str]] = None) -> Dict[int, Dict[str, Dict[str, float]]]:
    """{step: {key: {"min", "max", "mean", "ranks"}}} over all ``metrics.rank*.jsonl`` files in ``directory``."""
    per: Dict[int, Dict[str, List[float]]] = {}
    for fn in sorted(os.listdir(directory)):
        if not (fn.startswith("metrics.rank") and fn.endswith(".jsonl")):
            continue
        for line in open(os.path.join(directory, fn)):
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            slot = per.setdefault(int(rec["step"]), {})
            for k, v in rec.items():
                if k in ("t", "rank", "step") or not isinstance(v, (int, float)):
                    continue
                if keys is not None and k not in keys:
                    continue
                slot.setdefault(k, []).append(float(v))
    return {s: {k: {"min": min(v), "max": max(v), "mean": sum(v) / len(v), "ranks": len(v)} for k, v in d.items()}
            for s, d in sorted(per.items())}
