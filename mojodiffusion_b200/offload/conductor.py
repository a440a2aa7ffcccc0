"""Scalar policy that turns the trainer's offload switches into byte targets: activation offload and layer offload are
only active under CPU_OFFLOADED gradient checkpointing; ``layer_offload_fraction`` f keeps int(total * (1 - f)) bytes of
block weights on the device (serenitymojo/offload/conductor_policy.mojo:9-59)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence


@dataclass(frozen=True)
class ConductorPolicy:
    checkpointing_offload: bool
    activation_offload: bool
    layer_offload: bool
    async_transfer: bool
    layer_offload_fraction: float
    total_layer_bytes: int
    target_loaded_bytes: int

    @property
    def target_offloaded_bytes(self) -> int:
        return self.total_layer_bytes - self.target_loaded_bytes

    @property
    def needs_runtime_conductor(self) -> bool:
        return self.activation_offload or self.layer_offload


def conductor_policy(gradient_checkpointing: str, enable_activation_offloading: bool, enable_async_offloading: bool,
                     layer_offload_fraction: float, is_cuda: bool, total_layer_bytes: int) -> ConductorPolicy:
    if total_layer_bytes < 0:
        raise ValueError("total_layer_bytes must be non-negative")
    if not 0.0 <= layer_offload_fraction <= 1.0:
        raise ValueError("layer_offload_fraction must be within 0..1")
    ck = gradient_checkpointing.upper() == "CPU_OFFLOADED"
    layer = ck and layer_offload_fraction > 0.0
    loaded = int(total_layer_bytes * (1.0 - layer_offload_fraction)) if layer else total_layer_bytes
    return ConductorPolicy(ck, ck and enable_activation_offloading, layer, is_cuda and enable_async_offloading,
                           layer_offload_fraction, total_layer_bytes, loaded)


def resident_prefix(block_bytes: Sequence[int], budget_bytes: int) -> int:
    """Number of leading blocks that fit in ``budget_bytes`` (they stay on the device; the rest stream)."""
    used = n = 0
    for b in block_bytes:
        if used + b > budget_bytes:
            break
        used += b
        n += 1
    return n
