"""Block-swap weight streaming.

``PinnedBlockStore`` packs every block's tensors once into one page-locked host slab per block (256-byte aligned
members), so a block visit is ONE host->device DMA. ``BlockSwapLoader`` owns ``slot_count`` device slabs sized for the
largest block, a dedicated copy stream and two events per slot:

    ready[s]  recorded on the copy stream after the block's copy   -> the compute stream waits on it in await_block
    free[s]   recorded on the compute stream in mark_done          -> the copy stream waits on it before reusing s

so copies of block i+1 overlap the compute of block i without any host synchronisation. Blocks that fit a byte budget
can be pinned on the device permanently (``pin_residents``); they never take a slot. With 180 GB of HBM the usual
setting on this hardware is "everything resident"; streaming is for models or model zoos larger than that, and for
full fine-tunes whose optimizer state takes the room.

On a CPU device the same API runs with synchronous copies (used by the unit tests)
(serenitymojo/offload/block_loader.mojo:73-155, turbo_loader.mojo:157-670, turbo_planned_loader.mojo:91-447,
turbo_slots.mojo)."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .plan import BlockPlan
from .telemetry import OffloadTelemetry

ALIGN = 256


@dataclass(frozen=True)
class Member:
    name: str
    offset: int
    shape: Tuple[int, ...]
    dtype: torch.dtype
    nbytes: int


class PinnedBlockStore:
    def __init__(self, plan: BlockPlan, tensors: Mapping[str, torch.Tensor], pin: bool = True,
                 telemetry: Optional[OffloadTelemetry] = None):
        self.plan = plan
        self.telemetry = telemetry or OffloadTelemetry()
        t0 = time.perf_counter_ns()
        assign = plan.assign(tensors.keys())
        self.members: List[List[Member]] = []
        self.slabs: List[torch.Tensor] = []
        pin = pin and torch.cuda.is_available()
        for b in plan.blocks:
            names = assign[b.index]
            if not names:
                raise KeyError(f"block {b.index} ('{b.prefix}') matches no tensor")
            off, mem = 0, []
            for n in names:
                t = tensors[n]
                dt = torch.bfloat16 if (plan.config.dtype_policy == "force_bf16" and t.is_floating_point()
                                        and t.element_size() > 1) else t.dtype
                nb = t.numel() * torch.empty((), dtype=dt).element_size()
                mem.append(Member(n, off, tuple(t.shape), dt, nb))
                off = (off + nb + ALIGN - 1) // ALIGN * ALIGN
            slab = torch.empty(max(off, ALIGN), dtype=torch.uint8, pin_memory=pin)
            for m in mem:
                src = tensors[m.name].detach().to("cpu", m.dtype).contiguous()
                slab[m.offset:m.offset + m.nbytes].copy_(src.view(-1).view(torch.uint8))
            self.members.append(mem)
            self.slabs.append(slab)
        self.telemetry.pack_ns += time.perf_counter_ns() - t0

    def block_bytes(self) -> List[int]:
        return [s.numel() for s in self.slabs]

    def max_block_bytes(self) -> int:
        return max(self.block_bytes())

    def total_bytes(self) -> int:
        return sum(self.block_bytes())


def _views(slab: torch.Tensor, members: Sequence[Member]) -> Dict[str, torch.Tensor]:
    out = {}
    for m in members:
        out[m.name] = slab[m.offset:m.offset + m.nbytes].view(m.dtype).view(m.shape)
    return out


class BlockSwapLoader:
    def __init__(self, store: PinnedBlockStore, device, slot_count: Optional[int] = None, copy_stream_priority: int = 0):
        """``copy_stream_priority``: CUDA priority of the copy stream (0 default, -1 high). The race tests run every streamed
        workload under both and require bit-identical results: an ordering that only holds by scheduling luck shows up."""
        self.store, self.plan = store, store.plan
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.tel = store.telemetry
        n_slots = slot_count or self.plan.config.slot_count
        cap = store.max_block_bytes()
        self.slots = [torch.empty(cap, dtype=torch.uint8, device=self.device) for _ in range(n_slots)]
        self.slot_block: List[Optional[int]] = [None] * n_slots
        self.slot_busy: List[bool] = [False] * n_slots              # handed out by await_block, not yet mark_done
        self.slot_age: List[int] = [0] * n_slots
        self._clock = 0
        self.resident: Dict[int, torch.Tensor] = {}
        if self.cuda:
            self.copy_stream = torch.cuda.Stream(self.device, priority=copy_stream_priority)
            self.ready = [torch.cuda.Event() for _ in range(n_slots)]
            self.free = [torch.cuda.Event() for _ in range(n_slots)]
            self._free_recorded = [False] * n_slots

    # ---- permanent residents ----------------------------------------------------------------------------------
    def pin_residents(self, budget_bytes: int) -> int:
        """Keeps the first blocks that fit ``budget_bytes`` on the device for good. Returns how many."""
        used = n = 0
        for i, slab in enumerate(self.store.slabs):
            if used + slab.numel() > budget_bytes:
                break
            self.resident[i] = slab.to(self.device, non_blocking=False)
            used += slab.numel()
            n += 1
        return n

    # ---- slots -------------------------------------------------------------------------------------------------
    def _slot_of(self, block: int) -> Optional[int]:
        for s, b in enumerate(self.slot_block):
            if b == block:
                return s
        return None

    def _pick_slot(self) -> int:
        free = [s for s in range(len(self.slots)) if not self.slot_busy[s]]
        if not free:
            raise RuntimeError("block-swap: every slot is in use; call mark_done on a finished block first")
        empty = [s for s in free if self.slot_block[s] is None]
        return empty[0] if empty else min(free, key=lambda s: self.slot_age[s])

    def _issue_copy(self, block: int, slot: int) -> None:
        src = self.store.slabs[block]
        dst = self.slots[slot][:src.numel()]
        if self.cuda:
            with torch.cuda.stream(self.copy_stream):
                if self._free_recorded[slot]:
                    self.copy_stream.wait_event(self.free[slot])   # the previous tenant's compute has finished
                dst.copy_(src, non_blocking=True)
                self.ready[slot].record(self.copy_stream)
        else:
            dst.copy_(src)
        self.slot_block[slot] = block
        self._clock += 1
        self.slot_age[slot] = self._clock
        self.tel.h2d_bytes += src.numel()
        self.tel.h2d_copies += 1

    def prefetch(self, block: int) -> bool:
        """Starts the copy of ``block`` if it is neither resident nor already in a slot. Returns False when no slot is
        free right now (the caller simply awaits later)."""
        self.tel.prefetch_calls += 1
        if block in self.resident or self._slot_of(block) is not None:
            return True
        if all(self.slot_busy):
            return False
        self._issue_copy(block, self._pick_slot())
        return True

    def await_block(self, block: int) -> Dict[str, torch.Tensor]:
        """Tensor views of ``block`` on the device, valid until ``mark_done(block)``. The compute stream (the current
        stream) is made to wait for the copy; the host does not block."""
        self.tel.await_calls += 1
        if block in self.resident:
            self.tel.resident_hits += 1
            return _views(self.resident[block], self.store.members[block])
        slot = self._slot_of(block)
        if slot is None:
            self.tel.await_misses += 1
            slot = self._pick_slot()
            self._issue_copy(block, slot)
        else:
            self.tel.await_hits += 1
        if self.cuda:
            t0 = time.perf_counter_ns()
            torch.cuda.current_stream(self.device).wait_event(self.ready[slot])
            self.tel.await_wait_ns += time.perf_counter_ns() - t0
        self.slot_busy[slot] = True
        n = self.store.slabs[block].numel()
        return _views(self.slots[slot][:n], self.store.members[block])

    def mark_done(self, block: int) -> None:
        """The block's kernels have been enqueued; its slot may be overwritten once they finish."""
        if block in self.resident:
            return
        slot = self._slot_of(block)
        if slot is None or not self.slot_busy[slot]:
            raise RuntimeError(f"block-swap: mark_done({block}) without a matching await_block")
        if self.cuda:
            self.free[slot].record(torch.cuda.current_stream(self.device))
            self._free_recorded[slot] = True
        self.slot_busy[slot] = False

    def prefetch_next(self, block: int, reverse: bool = False) -> None:
        for j in self.plan.prefetch_targets(block, reverse):
            self.prefetch(j)


def guard_raw_copy_dtypes(members: Sequence[Member], expect: Mapping[str, torch.dtype]) -> None:
    """Raw byte copies reinterpret storage: refuse to hand a block to code that expects other dtypes."""
    for m in members:
        if m.name in expect and expect[m.name] != m.dtype:
            raise TypeError(f"{m.name}: stored as {m.dtype}, consumer expects {expect[m.name]}")
