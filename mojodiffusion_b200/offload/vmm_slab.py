"""Blocks of weights at fixed device addresses whose physical memory comes and goes.

``VmmSlab`` reserves one address range for all blocks of a model. A resident block is backed by physical memory; an evicted
one keeps its address but holds none. Because addresses never change, tensor views, tensor-map descriptors and captured
CUDA graphs built against a block stay valid across evict / reload cycles: only the bytes have to be copied in again. A
byte budget and reference counts drive eviction (least recently used first, blocks in use are never evicted).

Plays the role of the reference's serenitymojo/offload/vmm_slab.mojo:44-171 (reserve VA, create / map / unmap per block,
refcount, evict); the driver calls live in ``csrc/vmm_slab.cpp``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..ops import native


class VmmSlab:
    def __init__(self, block_bytes: Sequence[int], budget_bytes: Optional[int] = None, device: Optional[int] = None):
        native.load(True)
        self.o = native.ops()
        self.device = torch.cuda.current_device() if device is None else device
        self.gran = int(self.o.vmm_granularity(self.device))
        self.sizes = [(-(-int(b) // self.gran)) * self.gran for b in block_bytes]      # rounded to the granularity
        self.requested = [int(b) for b in block_bytes]
        self.offsets: List[int] = []
        off = 0
        for s in self.sizes:
            self.offsets.append(off)
            off += s
        self.handle = int(self.o.vmm_slab_create(off, self.device))
        self.budget = budget_bytes
        self.refs: Dict[int, int] = {}
        self.lru: List[int] = []                 # resident blocks, least recently used first
        self.loads = self.evictions = 0

    # ---- residency -------------------------------------------------------------------------------------------------------
    @property
    def resident_bytes(self) -> int:
        return int(self.o.vmm_slab_info(self.handle)[3])

    def is_resident(self, i: int) -> bool:
        return i in self.lru

    def address(self, i: int) -> int:
        return int(self.o.vmm_slab_info(self.handle)[0]) + self.offsets[i]

    def ensure_resident(self, i: int) -> bool:
        """Back block ``i`` with memory (evicting idle blocks if the budget needs it). Returns True when the block was NOT
        resident before, i.e. its bytes must be copied in by the caller."""
        if i in self.lru:
            self.lru.remove(i)
            self.lru.append(i)
            return False
        if self.budget is not None:
            while self.lru and self.resident_bytes + self.sizes[i] > self.budget:
                victim = next((b for b in self.lru if self.refs.get(b, 0) == 0), None)
                if victim is None:
                    raise MemoryError("VmmSlab: every resident block is in use and the budget is exhausted")
                self.evict(victim)
        self.o.vmm_slab_map(self.handle, self.offsets[i], self.sizes[i])
        self.lru.append(i)
        self.loads += 1
        return True

    def evict(self, i: int) -> None:
        """Release block ``i``'s memory. The caller has synchronised with every stream that may still read it."""
        if self.refs.get(i, 0) > 0:
            raise RuntimeError(f"VmmSlab: block {i} is in use")
        self.o.vmm_slab_unmap(self.handle, self.offsets[i])
        self.lru.remove(i)
        self.evictions += 1

    def acquire(self, i: int) -> torch.Tensor:
        """Pin block ``i`` (resident until ``release``) and return its bytes as a uint8 tensor."""
        self.ensure_resident(i)
        self.refs[i] = self.refs.get(i, 0) + 1
        return self.tensor(i)

    def release(self, i: int) -> None:
        assert self.refs.get(i, 0) > 0
        self.refs[i] -= 1

    def tensor(self, i: int, dtype=torch.uint8) -> torch.Tensor:
        t = self.o.vmm_slab_tensor(self.handle, self.offsets[i], self.requested[i])
        return t if dtype == torch.uint8 else t.view(dtype)

    def close(self) -> None:
        if self.handle:
            self.o.vmm_slab_destroy(self.handle)
            self.handle = 0
            self.lru.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
