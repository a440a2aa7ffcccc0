"""Metadata-only block plans: which weight prefixes form one streamed block, in which order they are visited, how many
branches visit each block per step (CFG-paired runs cond and uncond through a block before moving on), dtype policy and
prefetch lookahead. Nothing here touches a device (serenitymojo/offload/plan.mojo:9-318 and the per-model
``*_plan.mojo`` builders)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence

KINDS = ("transformer", "double_stream", "single_stream", "unet_down", "unet_mid", "unet_up")


@dataclass(frozen=True)
class OffloadConfig:
    slot_count: int = 2
    lookahead: int = 1
    dtype_policy: str = "preserve"            # preserve | force_bf16
    branch_schedule: str = "single"           # single | cfg_paired

    @property
    def branch_count(self) -> int:
        return 2 if self.branch_schedule == "cfg_paired" else 1

    def validate(self) -> None:
        if self.slot_count < 1 or self.lookahead < 0:
            raise ValueError("slot_count >= 1 and lookahead >= 0 required")
        if self.lookahead >= self.slot_count and self.slot_count > 1:
            raise ValueError("lookahead must be smaller than slot_count (a slot is needed for the block in use)")
        if self.dtype_policy not in ("preserve", "force_bf16") or self.branch_schedule not in ("single", "cfg_paired"):
            raise ValueError("unknown dtype policy or branch schedule")

    @staticmethod
    def single_pass():
        return OffloadConfig(1, 0)

    @staticmethod
    def double_buffered(cfg_paired: bool = False):
        return OffloadConfig(2, 1, "preserve", "cfg_paired" if cfg_paired else "single")


@dataclass(frozen=True)
class BlockSpec:
    index: int
    prefix: str                # every tensor whose name starts with this prefix belongs to the block
    kind: str = "transformer"


@dataclass
class BlockPlan:
    model: str
    blocks: List[BlockSpec]
    config: OffloadConfig = field(default_factory=OffloadConfig)

    def __len__(self):
        return len(self.blocks)

    def visit_order(self, reverse: bool = False) -> List[int]:
        """Block index per visit of one model evaluation (each block appears branch_count times in a row)."""
        idx = [b.index for b in self.blocks]
        if reverse:
            idx = idx[::-1]
        return [i for i in idx for _ in range(self.config.branch_count)]

    def next_block(self, i: int, reverse: bool = False, wrap: bool = True) -> Optional[int]:
        n = len(self.blocks)
        j = i - 1 if reverse else i + 1
        if 0 <= j < n:
            return j
        return (n - 1 if reverse else 0) if wrap else None

    def prefetch_targets(self, i: int, reverse: bool = False, wrap: bool = True) -> List[int]:
        out, j = [], i
        for _ in range(self.config.lookahead):
            j = self.next_block(j, reverse, wrap)
            if j is None or j == i:
                break
            out.append(j)
        return out

    def assign(self, names: Iterable[str]) -> Dict[int, List[str]]:
        """Tensor names per block. A name matching several prefixes goes to the longest one."""
        out: Dict[int, List[str]] = {b.index: [] for b in self.blocks}
        by_len = sorted(self.blocks, key=lambda b: -len(b.prefix))
        for n in names:
            for b in by_len:
                if n.startswith(b.prefix):
                    out[b.index].append(n)
                    break
        return out


def _seq(model, groups: Sequence, config) -> BlockPlan:
    blocks = []
    for fmt, count, kind in groups:
        for i in range(count):
            blocks.append(BlockSpec(len(blocks), fmt.format(i), kind))
    return BlockPlan(model, blocks, config or OffloadConfig())


def flux_plan(depth_double=19, depth_single=38, config=None):
    return _seq("flux", [("double_blocks.{}.", depth_double, "double_stream"), ("single_blocks.{}.", depth_single, "single_stream")], config)


def chroma_plan(config=None):
    return _seq("chroma", [("double_blocks.{}.", 19, "double_stream"), ("single_blocks.{}.", 38, "single_stream")], config)


def klein_plan(depth_double=8, depth_single=24, config=None):
    return _seq("klein", [("double_blocks.{}.", depth_double, "double_stream"), ("single_blocks.{}.", depth_single, "single_stream")], config)


def qwenimage_plan(depth=60, config=None):
    return _seq("qwenimage", [("transformer_blocks.{}.", depth, "double_stream")], config or OffloadConfig.double_buffered(True))


def zimage_plan(depth=30, refiners=2, config=None):
    return _seq("zimage", [("noise_refiner.{}.", refiners, "transformer"), ("context_refiner.{}.", refiners, "transformer"),
                           ("layers.{}.", depth, "transformer")], config)


def sd35_plan(depth=24, config=None):
    return _seq("sd35", [("joint_blocks.{}.", depth, "double_stream")], config)


def ltx2_plan(depth=48, config=None):
    return _seq("ltx2", [("transformer_blocks.{}.", depth, "transformer")], config)


def wan22_plan(depth=40, config=None):
    return _seq("wan22", [("blocks.{}.", depth, "transformer")], config)


def hidream_plan(depth_double=16, depth_single=32, config=None):
    return _seq("hidream", [("double_stream_blocks.{}.", depth_double, "double_stream"),
                            ("single_stream_blocks.{}.", depth_single, "single_stream")], config)


def l2p_plan(depth=30, config=None):
    return _seq("l2p", [("layers.{}.", depth, "transformer")], config)


def sdxl_plan(config=None):
    return _seq("sdxl", [("input_blocks.{}.", 9, "unet_down"), ("middle_block.", 1, "unet_mid"), ("output_blocks.{}.", 9, "unet_up")], config)


PLAN_BUILDERS = {"flux": flux_plan, "chroma": chroma_plan, "klein": klein_plan, "qwenimage": qwenimage_plan,
                 "zimage": zimage_plan, "sd35": sd35_plan, "ltx2": ltx2_plan, "wan22": wan22_plan,
                 "hidream": hidream_plan, "l2p": l2p_plan, "sdxl": sdxl_plan}


def plan_for(model: str, **kw) -> BlockPlan:
    if model not in PLAN_BUILDERS:
        raise KeyError(f"no offload plan for model '{model}'")
    return PLAN_BUILDERS[model](**kw)
