"""Residency bookkeeping for streamed blocks: a per-block state machine, a byte budget with high / low watermarks, and
an eviction order by next-use distance (the block whose next visit is farthest away goes first; pinned or in-use blocks
never go) (serenitymojo/offload/residency.mojo:40-526)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

UNLOADED, HOST_STAGED, PREFETCHING, GPU_READY, EVICTING, GPU_FREEING = (
    "unloaded", "host_staged", "prefetching", "gpu_ready", "evicting", "gpu_freeing")

_ALLOWED = {
    UNLOADED: {HOST_STAGED},
    HOST_STAGED: {PREFETCHING, UNLOADED},
    PREFETCHING: {GPU_READY, HOST_STAGED},
    GPU_READY: {EVICTING},
    EVICTING: {GPU_FREEING, GPU_READY},
    GPU_FREEING: {HOST_STAGED, UNLOADED},
}


def is_gpu_resident(state: str) -> bool:
    return state in (GPU_READY, EVICTING)


@dataclass
class ResidencyEntry:
    byte_count: int = 0
    state: str = UNLOADED
    refcount: int = 0
    pinned: bool = False
    last_visit: int = -1

    def can_evict(self) -> bool:
        return self.state == GPU_READY and self.refcount == 0 and not self.pinned


class BudgetTracker:
    def __init__(self, high_bytes: int, low_bytes: int):
        if low_bytes < 0 or high_bytes < low_bytes:
            raise ValueError("0 <= low_bytes <= high_bytes required")
        self.high, self.low, self.current = high_bytes, low_bytes, 0

    @property
    def headroom(self) -> int:
        return max(0, self.high - self.current)

    def above_high(self) -> bool:
        return self.current > self.high

    def below_low(self) -> bool:
        return self.current < self.low

    def can_prefetch(self, nbytes: int = 0) -> bool:
        return self.current + nbytes <= self.high

    def should_evict(self) -> bool:
        return self.current > self.high

    def add(self, n: int) -> None:
        self.current += n

    def remove(self, n: int) -> None:
        self.current = max(0, self.current - n)


class ResidencyManager:
    def __init__(self, block_bytes: Sequence[int], visit_order: Sequence[int], high_bytes: int, low_bytes: Optional[int] = None,
                 lookahead: int = 1):
        self.entries = [ResidencyEntry(b) for b in block_bytes]
        self.order = list(visit_order)
        self.budget = BudgetTracker(high_bytes, high_bytes * 3 // 4 if low_bytes is None else low_bytes)
        self.lookahead = lookahead

    def state(self, i: int) -> str:
        return self.entries[i].state

    def transition(self, i: int, new: str) -> None:
        e = self.entries[i]
        if new not in _ALLOWED[e.state]:
            raise RuntimeError(f"block {i}: illegal residency transition {e.state} -> {new}")
        if new == EVICTING and (e.refcount > 0 or e.pinned):
            raise RuntimeError(f"block {i}: cannot evict a block that is in use or pinned")
        was, now = is_gpu_resident(e.state) or e.state == PREFETCHING, is_gpu_resident(new) or new == PREFETCHING
        if now and not was:
            self.budget.add(e.byte_count)
        if was and not now and new != GPU_FREEING:
            self.budget.remove(e.byte_count)
        if new == GPU_FREEING:
            self.budget.remove(e.byte_count)
        e.state = new

    def acquire(self, i: int) -> None:
        if self.entries[i].state != GPU_READY:
            raise RuntimeError(f"block {i}: acquire needs gpu_ready, is {self.entries[i].state}")
        self.entries[i].refcount += 1

    def release(self, i: int) -> None:
        if self.entries[i].refcount <= 0:
            raise RuntimeError(f"block {i}: release without acquire")
        self.entries[i].refcount -= 1

    def pin(self, i: int, pinned: bool = True) -> None:
        self.entries[i].pinned = pinned

    def mark_visit(self, i: int, step: int) -> None:
        self.entries[i].last_visit = step

    def next_use_distance(self, block: int, cursor: int) -> int:
        """Visits from position ``cursor`` of the (cyclic) visit order until ``block`` is needed again."""
        n = len(self.order)
        for d in range(n):
            if self.order[(cursor + d) % n] == block:
                return d
        return n + 1                                  # never visited: evict first

    def eviction_order(self, cursor: int) -> List[int]:
        cand = [i for i, e in enumerate(self.entries) if e.can_evict()]
        return sorted(cand, key=lambda i: (-self.next_use_distance(i, cursor), i))

    def blocks_to_evict(self, cursor: int, incoming_bytes: int = 0) -> List[int]:
        """Evict (farthest next use first) until current + incoming fits under the high watermark; once eviction
        starts it continues down to the low watermark to avoid thrashing."""
        if self.budget.current + incoming_bytes <= self.budget.high:
            return []
        out, cur = [], self.budget.current + incoming_bytes
        for i in self.eviction_order(cursor):
            if cur <= self.budget.low:
                break
            out.append(i)
            cur -= self.entries[i].byte_count
        return out

    def prefetch_targets(self, cursor: int) -> List[int]:
        n = len(self.order)
        out = []
        for d in range(1, self.lookahead + 1):
            b = self.order[(cursor + d) % n]
            e = self.entries[b]
            if e.state in (UNLOADED, HOST_STAGED) and b not in out and self.budget.can_prefetch(e.byte_count):
                out.append(b)
        return out
