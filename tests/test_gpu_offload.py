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


def test_vmm_slab_keeps_addresses_while_physical_memory_comes_and_goes():
    """Blocks keep their device address across evict / reload; a byte budget evicts the least recently used idle block;
    blocks in use are never evicted; a captured CUDA graph that reads a block sees the bytes loaded after a reload.
    Unmapped ranges are never touched: views of them are refused on the host."""
    import pytest
    import torch
    from mojodiffusion_b200.offload.vmm_slab import VmmSlab
    MiB = 1 << 20
    slab = VmmSlab([3 * MiB] * 4, budget_bytes=2 * 4 * MiB)
    try:
        assert slab.gran % (64 * 1024) == 0 and all(s % slab.gran == 0 and s >= 3 * MiB for s in slab.sizes)
        free0 = torch.cuda.mem_get_info()[0]
        addr = [slab.address(i) for i in range(4)]
        a = slab.acquire(0)
        assert a.numel() == 3 * MiB and a.data_ptr() == addr[0]
        a.fill_(7)
        slab.release(0)
        assert slab.ensure_resident(1) is True and slab.ensure_resident(1) is False
        slab.tensor(1).fill_(9)
        torch.cuda.synchronize()
        assert slab.resident_bytes == 2 * slab.sizes[0] and free0 - torch.cuda.mem_get_info()[0] >= 2 * slab.sizes[0] - MiB
        assert slab.ensure_resident(2) is True                      # over budget: block 0 (least recently used) goes
        assert not slab.is_resident(0) and slab.is_resident(1) and slab.is_resident(2) and slab.evictions == 1
        with pytest.raises(RuntimeError):
            slab.tensor(0)                                          # a view of an unmapped range is refused
        assert [slab.address(i) for i in range(4)] == addr
        assert int(slab.tensor(1)[12345]) == 9
        # a block in use is never the victim
        t2 = slab.acquire(2)
        assert slab.ensure_resident(3) is True and slab.is_resident(2) and not slab.is_resident(1)
        t3 = slab.acquire(3)
        with pytest.raises(MemoryError):
            slab.ensure_resident(0)
        slab.release(3)
        slab.release(2)
        # CUDA graph over a fixed address: reload the block with other bytes, replay, see the new bytes
        x = slab.tensor(2, torch.float32)
        x.fill_(1.5)
        out = torch.zeros(1, device="cuda")
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            out.copy_(x[:1024].sum().reshape(1))                    # warm-up outside capture
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out.copy_(x[:1024].sum().reshape(1))
        g.replay()
        torch.cuda.synchronize()
        assert float(out) == 1.5 * 1024
        del x, t2, t3
        slab.evict(2)
        assert slab.ensure_resident(2) is True and slab.address(2) == addr[2]
        slab.tensor(2, torch.float32).fill_(2.0)
        g.replay()
        torch.cuda.synchronize()
        assert float(out) == 2.0 * 1024
        with pytest.raises(RuntimeError):
            torch.ops.mdb200.vmm_slab_map(slab.handle, slab.offsets[2], slab.sizes[2])     # overlaps a mapped region
    finally:
        torch.cuda.synchronize()
        slab.close()


def test_fsdp_optimizer_state_offload_matches_device_resident_state():
    """Sharded linears with their fp32 masters and AdamW moments in pinned host memory, streamed through device staging slots
    per step: after several training steps the master shards, the moments and the bf16 weight shards equal those of the
    same run with device-resident state bit for bit (one process: the sharding degenerates to one shard per layer)."""
    from mojodiffusion_b200.parallel.fsdp import FSDPContext, FSDPLinear

    def run(offload):
        ctx = FSDPContext(mode="fused", offload_optimizer=offload)
        dims = [(256, 512), (512, 1024), (1024, 256), (256, 128)]
        layers = [FSDPLinear(ctx, i, o, bias=False, seed=10 + k) for k, (i, o) in enumerate(dims)]
        ctx.finalize()
        g = torch.Generator().manual_seed(0)
        for step in range(3):
            x = torch.randn(64, 256, generator=g).to("cuda", torch.bfloat16)
            h = x
            for l in layers:
                h = torch.tanh(l(h))
            h.float().square().mean().backward()
            ctx.step(lr=1e-2, weight_decay=0.1)
        torch.cuda.synchronize()
        ctx.check()
        return ctx, layers

    c0, l0 = run(False)
    c1, l1 = run(True)
    assert all(not l.master.is_cuda and l.master.is_pinned() and not l.m.is_cuda for l in l1)
    for a, b in zip(l0, l1):
        assert torch.equal(a.master.cpu(), b.master) and torch.equal(a.m.cpu(), b.m) and torch.equal(a.v.cpu(), b.v)
        assert torch.equal(a.w_shard, b.w_shard)
        assert float(b.m.abs().sum()) > 0 and torch.equal(b.full_master().cpu(), b.master)
