"""Offload: plan / residency / conductor contracts without a device, and the block-swap loader + streamed stack on the
CPU device (synchronous copies, same bookkeeping)."""
import pytest
import torch
from torch import nn

from mojodiffusion_b200.offload import (BlockSwapLoader, OffloadConfig, PinnedBlockStore, ResidencyManager, StreamedStack,
                                        conductor_policy, plan_for, resident_prefix)
from mojodiffusion_b200.offload import residency as R
from mojodiffusion_b200.offload.loader import guard_raw_copy_dtypes
from mojodiffusion_b200.offload.plan import BlockPlan, BlockSpec


def test_plans():
    p = plan_for("flux")
    assert len(p) == 57 and p.blocks[0].prefix == "double_blocks.0." and p.blocks[19].kind == "single_stream"
    assert p.next_block(56) == 0 and p.next_block(0, reverse=True) == 56 and p.next_block(56, wrap=False) is None
    q = plan_for("qwenimage")
    assert len(q) == 60 and q.config.branch_count == 2 and q.visit_order()[:4] == [0, 0, 1, 1]
    assert q.visit_order(reverse=True)[:2] == [59, 59]
    names = ["double_blocks.1.img_attn.qkv.weight", "double_blocks.10.img_attn.qkv.weight", "img_in.weight"]
    a = p.assign(names)
    assert a[1] == [names[0]] and a[10] == [names[1]] and sum(len(v) for v in a.values()) == 2
    with pytest.raises(ValueError):
        OffloadConfig(2, 2).validate()
    with pytest.raises(KeyError):
        plan_for("nope")
    for m in ("chroma", "klein", "zimage", "sd35", "ltx2", "wan22", "hidream", "l2p", "sdxl"):
        assert len(plan_for(m)) > 0


def test_residency_fsm_budget_and_eviction():
    m = ResidencyManager([100] * 5, [0, 1, 2, 3, 4], high_bytes=300, low_bytes=200, lookahead=1)
    with pytest.raises(RuntimeError):
        m.transition(0, R.GPU_READY)
    for i in (0, 1, 2):
        m.transition(i, R.HOST_STAGED)
        m.transition(i, R.PREFETCHING)
        m.transition(i, R.GPU_READY)
    assert m.budget.current == 300 and not m.budget.can_prefetch(100)
    m.acquire(1)
    # cursor at block 1: block 0 is needed farthest in the future (4 visits away), block 2 next
    assert m.next_use_distance(0, 1) == 4 and m.next_use_distance(2, 1) == 1
    assert m.eviction_order(1) == [0, 2]                     # block 1 is in use
    assert m.blocks_to_evict(1, incoming_bytes=100) == [0, 2][:2] or m.blocks_to_evict(1, 100) == [0]
    with pytest.raises(RuntimeError):
        m.transition(1, R.EVICTING)
    m.transition(0, R.EVICTING)
    m.transition(0, R.GPU_FREEING)
    m.transition(0, R.HOST_STAGED)
    assert m.budget.current == 200
    m.release(1)
    with pytest.raises(RuntimeError):
        m.release(1)
    m.pin(2)
    assert m.eviction_order(3) == [1]
    m.transition(3, R.HOST_STAGED)
    assert m.prefetch_targets(2) == [3]


def test_conductor_policy():
    p = conductor_policy("CPU_OFFLOADED", True, True, 0.25, True, 1000)
    assert p.layer_offload and p.activation_offload and p.async_transfer
    assert p.target_loaded_bytes == 750 and p.target_offloaded_bytes == 250 and p.needs_runtime_conductor
    q = conductor_policy("ON", True, True, 0.5, True, 1000)
    assert not q.layer_offload and q.target_loaded_bytes == 1000 and not q.needs_runtime_conductor
    with pytest.raises(ValueError):
        conductor_policy("ON", False, False, 1.5, False, 10)
    assert resident_prefix([10, 10, 10, 10], 25) == 2


class _Block(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(d, 2 * d), nn.Linear(2 * d, d)
        self.lora = nn.Parameter(torch.zeros(d, d))

    def forward(self, x):
        return x + self.fc2(torch.nn.functional.gelu(self.fc1(x))) + x @ self.lora


def _setup(n=5, d=8, slots=2):
    torch.manual_seed(0)
    blocks = nn.ModuleList([_Block(d) for _ in range(n)])
    for b in blocks:
        nn.init.normal_(b.lora, std=0.05)
    plan = BlockPlan("toy", [BlockSpec(i, f"blocks.{i}.") for i in range(n)], OffloadConfig(slots, 1))
    frozen = {f"blocks.{i}.{k}": v for i, b in enumerate(blocks) for k, v in b.state_dict().items() if "lora" not in k}
    return blocks, plan, frozen


def test_block_swap_loader_and_streamed_forward():
    blocks, plan, frozen = _setup()
    x = torch.randn(3, 8)
    ref = x
    for b in blocks:
        ref = b(ref)
    store = PinnedBlockStore(plan, frozen, pin=False)
    assert len(store.slabs) == 5 and all(m.offset % 256 == 0 for mem in store.members for m in mem)
    loader = BlockSwapLoader(store, "cpu")
    assert loader.pin_residents(store.block_bytes()[0] + 1) == 1
    stack = StreamedStack(list(blocks), loader)
    stack.detach_weights()
    assert blocks[2].fc1.weight.numel() == 0
    with torch.no_grad():
        out = stack.forward(lambda blk, h: blk(h), x)
        out2 = stack.forward(lambda blk, h: blk(h), x)       # second pass wraps around the slots
    assert torch.equal(out, ref.detach()) and torch.equal(out2, out)
    t = loader.tel
    assert t.resident_hits == 2 and t.await_calls == 10 and t.await_hits >= 6 and t.h2d_copies <= 9
    assert "hit_rate" in t.line()
    # slot discipline
    v = loader.await_block(1)
    loader.await_block(2)
    with pytest.raises(RuntimeError):
        loader.await_block(3)                                 # both slots handed out
    loader.mark_done(1)
    loader.mark_done(2)
    with pytest.raises(RuntimeError):
        loader.mark_done(2)
    with pytest.raises(TypeError):
        guard_raw_copy_dtypes(store.members[1], {"blocks.1.fc1.weight": torch.bfloat16})


def test_streamed_training_matches_resident_gradients():
    blocks, plan, frozen = _setup()
    x = torch.randn(3, 8, requires_grad=True)
    h = x
    for b in blocks:
        for n, p in b.named_parameters():
            p.requires_grad_("lora" in n)
        h = b(h)
    h.pow(2).mean().backward()
    ref_gx = x.grad.clone()
    ref_gl = [b.lora.grad.clone() for b in blocks]
    x.grad = None
    for b in blocks:
        b.lora.grad = None
    loader = BlockSwapLoader(PinnedBlockStore(plan, frozen, pin=False), "cpu")
    stack = StreamedStack(list(blocks), loader)
    stack.detach_weights()
    out = stack.forward_train(lambda blk, hh: blk(hh), x)
    out.pow(2).mean().backward()
    assert torch.allclose(x.grad, ref_gx, atol=1e-6)
    for b, g in zip(blocks, ref_gl):
        assert torch.allclose(b.lora.grad, g, atol=1e-6)
    assert loader.tel.await_calls == 10                      # every block streamed once forward, once backward


def test_parallel_video_dit_single_rank_equals_model():
    """The token-sharded video DiT driver with one rank (no communication) restates the model's forward exactly."""
    import torch
    from mojodiffusion_b200.models.video_dit import VideoDiT, tiny_video_dit_config
    from mojodiffusion_b200.parallel.video_parallel import ParallelVideoDiT
    cfg = tiny_video_dit_config()
    m = VideoDiT(cfg, torch.float32, "cpu").init_weights(0)
    with torch.no_grad():
        for blk in m.transformer_blocks:
            blk.scale_shift_table.copy_(0.1 * torch.randn(blk.scale_shift_table.shape, generator=torch.Generator().manual_seed(3)))
    g = torch.Generator().manual_seed(1)
    grid = (2, 4, 4)
    x = torch.randn(1, 32, cfg.in_channels, generator=g)
    ctx = torch.randn(1, 8, cfg.context_dim, generator=g)
    t = torch.tensor([0.6])

    par = ParallelVideoDiT(m, grid, mode="nccl", device=torch.device("cpu"))
    with torch.no_grad():
        want = m(x, ctx, t, grid)
        got = par.forward(x, ctx, t)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), float((got - want).abs().max())
