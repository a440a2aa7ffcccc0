"""Symmetric (peer-mapped) device buffers.

``SymmetricBuffer.create`` allocates a buffer through ``torch.distributed._symmetric_memory`` and exchanges the
mappings over the process group, so every rank holds a device address for every peer's copy (NVLink P2P) and, when
the fabric supports it, one NVLS multicast address that reaches all copies at once. The kernels in
``csrc/comm_kernels.cu`` and the peer-routed GEMM / attention epilogues take these raw addresses.

``emulated_group`` builds the same structure from N ordinary allocations on ONE GPU: the single-GPU tests drive
the multi-rank kernels with it, rank by rank, over all ranks' data (no kernel ever waits on another launch).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class SymmetricBuffer:
    local: torch.Tensor                 # uint8 view of this rank's copy
    peer_ptrs: List[int]                # device address of every rank's copy (index = rank)
    rank: int
    world: int
    mc_ptr: int = 0                     # NVLS multicast address (0: none)
    handle: object = None
    peers_local: Optional[List[torch.Tensor]] = None   # emulation only: the other ranks' tensors

    @staticmethod
    def create(nbytes: int, group=None, device=None, use_multicast: bool = True) -> "SymmetricBuffer":
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        nbytes = (nbytes + 255) // 256 * 256
        t = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        hdl = symm_mem.rendezvous(t, group)
        t.zero_()
        mc = 0
        if use_multicast:
            try:
                mc = int(hdl.multicast_ptr) if hdl.has_multicast_support else 0
            except Exception:
                mc = 0
        buf = SymmetricBuffer(t, [int(p) for p in hdl.buffer_ptrs], hdl.rank, hdl.world_size, mc, hdl)
        torch.cuda.synchronize(device)
        dist.barrier(group)
        return buf

    def view(self, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nb = numel * torch.empty(0, dtype=dtype).element_size()
        return self.local[offset:offset + nb].view(dtype)

    def ptrs_at(self, offset: int) -> List[int]:
        return [p + offset for p in self.peer_ptrs]

    def mc_at(self, offset: int) -> int:
        return self.mc_ptr + offset if self.mc_ptr else 0


def emulated_group(world: int, nbytes: int, device="cuda") -> List[SymmetricBuffer]:
    nbytes = (nbytes + 255) // 256 * 256
    ts = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
    ptrs = [t.data_ptr() for t in ts]
    return [SymmetricBuffer(ts[r], ptrs, r, world, 0, None, ts) for r in range(world)]
