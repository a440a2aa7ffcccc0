"""Loader of the in-tree native library.

The library is looked for next to the package (``mojodiffusion_b200/_C.so``). On a machine with a GPU a
missing library is an error on first use: the CUDA path is the product, and a silent fall-back to eager
PyTorch there would hide that it is not running. Without a GPU (unit tests on CPU) the pure-torch
references in ``ops.reference`` serve instead.
"""
from __future__ import annotations

import os
import threading
from pathlib import Path

import torch

_LIB = Path(__file__).resolve().parent.parent / "_C.so"
_lock = threading.Lock()
_loaded = False
_error: str | None = None


def lib_path() -> Path:
    return _LIB


def load(required: bool = False) -> bool:
    """Load ``_C.so`` once. Returns True when ``torch.ops.mdb200`` is usable."""
    global _loaded, _error
    if _loaded:
        return True
    with _lock:
        if _loaded:
            return True
        if not _LIB.exists():
            _error = f"{_LIB} not found: run `python -m mojodiffusion_b200._build`"
        else:
            try:
                torch.ops.load_library(str(_LIB))
                _loaded = True
                _error = None
            except Exception as e:  # pragma: no cover - depends on the machine
                _error = f"loading {_LIB} failed: {e}"
    if not _loaded and required:
        raise RuntimeError(f"mojodiffusion_b200 native kernels unavailable: {_error}")
    return _loaded


def available() -> bool:
    return load(False)


def ops():
    """``torch.ops.mdb200`` (raises if the library cannot be loaded)."""
    load(True)
    return torch.ops.mdb200


def use_native(t: torch.Tensor) -> bool:
    """True when `t` lives on a GPU; the native library is then mandatory."""
    if not t.is_cuda:
        return False
    if os.environ.get("MDB200_FORCE_REFERENCE") == "1":
        return False
    load(True)
    return True


def check_status(like: torch.Tensor | None = None, reset: bool = True) -> None:
    """Raise if any kernel since the last check abandoned a bounded wait (synchronises the device)."""
    if like is None:
        if not torch.cuda.is_available():
            return
        like = torch.empty(0, device="cuda")
    if not like.is_cuda or not available():
        return
    code, where, block, extra = ops().read_status(like, reset)
    if code != 0:
        names = {1: "TIMEOUT", 2: "BAD_ARG", 3: "BOUNDS"}
        raise RuntimeError(
            f"mdb200 kernel reported {names.get(code, code)} (where={where}, block={block}, extra={extra})")
