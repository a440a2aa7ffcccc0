"""Block-swap streaming on the GPU: streamed bytes equal resident bytes, streamed inference and LoRA training equal the
resident model, copies really overlap (hit rate)."""
import pytest
import torch

from mojodiffusion_b200.models.mmdit import MMDiT, tiny_mmdit_config
from mojodiffusion_b200.offload import BlockSwapLoader, PinnedBlockStore
from mojodiffusion_b200.offload.plan import flux_plan
from mojodiffusion_b200.ops import native
from mojodiffusion_b200.training.lora import collect_slots, inject_flux_lora, lora_parameters

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


def _model(seed=0):
    native.load(True)
    cfg = tiny_mmdit_config()
    m = MMDiT(cfg, torch.bfloat16, DEV)
    m.init_weights(seed)
    return m, cfg


def _inputs(cfg, B=1, S_img=256, S_txt=64):
    g = torch.Generator().manual_seed(1)
    img = torch.randn(B, S_img, cfg.in_channels, generator=g).to(DEV, torch.bfloat16)
    txt = torch.randn(B, S_txt, cfg.context_dim, generator=g).to(DEV, torch.bfloat16)
    y = torch.randn(B, cfg.vec_dim, generator=g).to(DEV, torch.bfloat16)
    t = torch.full((B,), 0.5, device=DEV)
    return img, txt, t, y


def test_streamed_bytes_equal_resident_bytes():
    m, cfg = _model()
    plan = flux_plan(cfg.depth_double, cfg.depth_single)
    blocks = list(m.double_blocks) + list(m.single_blocks)
    tensors = {s.prefix + n: p.detach() for s, b in zip(plan.blocks, blocks) for n, p in b.named_parameters()}
    loader = BlockSwapLoader(PinnedBlockStore(plan, tensors), DEV)
    for rep in range(2):
        for i in range(len(plan)):
            views = loader.await_block(i)
            loader.prefetch_next(i)
            for k, v in views.items():
                assert v.dtype == tensors[k].dtype and torch.equal(v, tensors[k]), k
            loader.mark_done(i)
    torch.cuda.synchronize()
    assert loader.tel.await_misses == 1 and loader.tel.h2d_bytes > 0      # only the very first block was not prefetched


def test_streamed_inference_and_lora_training_match_resident():
    m, cfg = _model()
    slots = inject_flux_lora(m, rank=8, alpha=8.0)
    for s in slots:
        with torch.no_grad():
            s.up.normal_(0, 0.02)
    for n, p in m.named_parameters():
        p.requires_grad_(".slots." in n)
    img, txt, t, y = _inputs(cfg)
    g = torch.ones(1, device=DEV) if cfg.guidance_embed else None
    with torch.no_grad():
        ref = m(img, txt, t, y, g)
    out = m(img, txt, t, y, g)
    out.float().pow(2).mean().backward()
    ref_grads = [p.grad.clone() for p in lora_parameters(slots)]
    for p in lora_parameters(slots):
        p.grad = None
    first = sum(p.numel() * p.element_size() for p in m.double_blocks[0].parameters())
    loader = m.enable_block_swap(DEV, resident_budget_bytes=first + 4096)
    assert len(loader.resident) == 1 and m.single_blocks[0].linear1.weight.numel() == 0
    with torch.no_grad():
        got = m(img, txt, t, y, g)
    assert torch.equal(got, ref)
    out2 = m(img, txt, t, y, g)
    out2.float().pow(2).mean().backward()
    for p, r in zip(lora_parameters(slots), ref_grads):
        assert p.grad is not None
        assert torch.allclose(p.grad.float(), r.float(), atol=1e-3, rtol=2e-2)
    torch.cuda.synchronize()
    native.check_status()
    assert loader.tel.await_calls >= 3 * (cfg.depth_double + cfg.depth_single)


def test_streaming_is_bit_identical_under_permuted_stream_priorities():
    """Race-detection substitute: the same streamed forward with the copy stream at default and at high priority, twice
    each, after the slots were filled with a poison pattern. Every result must be bit-identical to the resident model: a
    consumer that reads a slot before its copy landed (or a copy that overwrites a slot still in use) would differ."""
    m, cfg = _model()
    img, txt, t, y = _inputs(cfg)
    g = torch.ones(1, device=DEV) if cfg.guidance_embed else None
    with torch.no_grad():
        ref = m(img, txt, t, y, g)
    plan = flux_plan(cfg.depth_double, cfg.depth_single)
    blocks = list(m.double_blocks) + list(m.single_blocks)
    tensors = {s.prefix + n: p.detach().clone() for s, b in zip(plan.blocks, blocks) for n, p in b.named_parameters()}
    for prio in (0, -1, 0, -1):
        loader = BlockSwapLoader(PinnedBlockStore(plan, tensors), DEV, copy_stream_priority=prio)
        for s in loader.slots:
            s.fill_(0xFF)                                    # bf16 0xFFFF = NaN: any read of an unfilled slot poisons the output
        torch.cuda.synchronize()
        outs = []
        for rep in range(2):
            with torch.no_grad():
                # every block's weights reach it only through the loader's slots
                from mojodiffusion_b200.offload.streamed import StreamedStack
                m.streamer = StreamedStack(blocks, loader)
                try:
                    outs.append(m(img, txt, t, y, g))
                finally:
                    m.streamer = None
        torch.cuda.synchronize()
        for o in outs:
            assert torch.isfinite(o.float()).all() and torch.equal(o, ref), f"priority {prio}"
    native.check_status()
