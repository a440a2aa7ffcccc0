"""Process-group plumbing: one process per GPU, torch.distributed (NCCL on GPUs, gloo on CPU ranks)."""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist


def env_rank() -> int:
    return int(os.environ.get("RANK", "0"))


def env_world() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def env_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def init_from_env(backend: Optional[str] = None, timeout_s: float = 600.0) -> bool:
    """Initialise the default group from RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT. Returns True if
    a multi-rank group exists afterwards."""
    if dist.is_initialized():
        return dist.get_world_size() > 1
    if env_world() <= 1:
        return False
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(env_local_rank())
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s),
                                device_id=torch.device("cuda", env_local_rank()))
    else:
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s))
    return True


def world_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def barrier(group=None) -> None:
    if dist.is_initialized():
        if torch.cuda.is_available() and dist.get_backend(group) == "nccl":
            dist.barrier(group, device_ids=[torch.cuda.current_device()])
        else:
            dist.barrier(group)


def max_over_ranks(value: float, group=None) -> float:
    """Max of a host scalar over all ranks (device-timed numbers are reported as the slowest rank's)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
