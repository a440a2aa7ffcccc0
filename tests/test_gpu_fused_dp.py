"""Fused data-parallel path (reduce-scatter + clip + AdamW + all-gather in peer-memory kernels).

On one GPU the N ranks are emulated over N buffers of the same device, phase by phase (no launch waits on
another launch). With two or more GPUs the same class runs as real ranks over NVLink and must agree with the
NCCL all-reduce baseline."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(params0, grads_per_rank, steps, lr, wd, max_norm):
    ps = [p.float().clone() for p in params0]
    ms = [torch.zeros_like(p) for p in ps]
    vs = [torch.zeros_like(p) for p in ps]
    world = len(grads_per_rank[0])
    for t in range(steps):
        gs = [sum(g[i].float() for g in grads_per_rank[t]) / world for i in range(len(ps))]
        norm = torch.sqrt(sum((g ** 2).sum() for g in gs))
        clip = min(1.0, max_norm / (float(norm) + 1e-6)) if max_norm > 0 else 1.0
        for i in range(len(ps)):
            g = gs[i] * clip
            p = ps[i].bfloat16().float() * (1 - lr * wd)
            ms[i] = 0.9 * ms[i] + 0.1 * g
            vs[i] = 0.999 * vs[i] + 0.001 * g * g
            p = p - (lr / (1 - 0.9 ** (t + 1))) * (ms[i] / (vs[i].sqrt() / (1 - 0.999 ** (t + 1)) ** 0.5 + 1e-8))
            ps[i] = p.bfloat16().float()
    return ps


def test_emulated_ranks_match_reference():
    from mojodiffusion_b200.ops import native
    from mojodiffusion_b200.parallel.fused_dp import emulate_ranks, emulated_step
    dev = "cuda"
    world, steps, lr, wd, max_norm = 4, 3, 1e-2, 0.01, 1.0
    shapes = [(16, 3072), (3072, 16), (7,), (1000, 33)]
    g = torch.Generator().manual_seed(0)
    base = [torch.randn(*s, generator=g).bfloat16() for s in shapes]
    sets = [[torch.nn.Parameter(b.clone().to(dev)) for b in base] for _ in range(world)]
    ranks = emulate_ranks(sets, lr=lr, weight_decay=wd, max_grad_norm=max_norm)
    grads = [[[torch.randn(*s, generator=g).bfloat16() for s in shapes] for _ in range(world)] for _ in range(steps)]
    for t in range(steps):
        for r in range(world):
            ranks[r].zero_grad()
            for p, gg in zip(sets[r], grads[t][r]):
                p.grad.copy_(gg.to(dev))
        emulated_step(ranks)
    torch.cuda.synchronize()
    native.check_status()
    want = _reference(base, grads, steps, lr, wd, max_norm)
    for r in range(world):
        for p, w in zip(sets[r], want):
            assert torch.allclose(p.detach().float().cpu(), w, atol=2e-2, rtol=2e-2)
    for r in range(1, world):  # replicas stay bit-identical
        for a, b in zip(sets[0], sets[r]):
            assert torch.equal(a.detach(), b.detach())
    assert abs(ranks[0].grad_norm() - ranks[1].grad_norm()) < 1e-6


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _mp_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from mojodiffusion_b200.ops import native
    from mojodiffusion_b200.parallel.fused_dp import FusedDPAdamW
    dev = torch.device("cuda", rank)
    shapes = [(16, 3072), (3072, 16), (7,), (1000, 33)]
    g = torch.Generator().manual_seed(0)
    base = [torch.randn(*s, generator=g).bfloat16() for s in shapes]
    for use_mc in (False, True):
        params = [torch.nn.Parameter(b.clone().to(dev)) for b in base]
        refp = [b.clone().to(dev).float() for b in base]
        opt = FusedDPAdamW(params, lr=1e-2, weight_decay=0.01, max_grad_norm=1.0, use_multicast=use_mc)
        gg = torch.Generator().manual_seed(100 + rank)
        ms = [torch.zeros_like(p) for p in refp]
        vs = [torch.zeros_like(p) for p in refp]
        for t in range(3):
            opt.zero_grad()
            gl = [torch.randn(*s, generator=gg).bfloat16().to(dev) for s in shapes]
            for p, x in zip(params, gl):
                p.grad.copy_(x)
            opt.step()
            # NCCL baseline of the same step
            red = [x.float() for x in gl]
            for x in red:
                dist.all_reduce(x)
                x /= world
            norm = torch.sqrt(sum((x ** 2).sum() for x in red))
            clip = min(1.0, 1.0 / (float(norm) + 1e-6))
            for i in range(len(refp)):
                x = red[i] * clip
                p = refp[i].bfloat16().float() * (1 - 1e-2 * 0.01)
                ms[i] = 0.9 * ms[i] + 0.1 * x
                vs[i] = 0.999 * vs[i] + 0.001 * x * x
                p = p - (1e-2 / (1 - 0.9 ** (t + 1))) * (ms[i] / (vs[i].sqrt() / (1 - 0.999 ** (t + 1)) ** 0.5 + 1e-8))
                refp[i] = p.bfloat16().float()
        torch.cuda.synchronize()
        native.check_status()
        for p, w in zip(params, refp):
            assert torch.allclose(p.detach().float(), w, atol=2e-2, rtol=2e-2), f"rank {rank} mc={use_mc}"
        chk = torch.stack([p.detach().float().sum() for p in params])
        allc = [torch.empty_like(chk) for _ in range(world)]
        dist.all_gather(allc, chk)
        assert all(torch.equal(allc[0], c) for c in allc), "replicas diverged"
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        open(os.path.join(out_dir, "ok"), "w").write("ok")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_real_ranks_match_nccl_baseline(tmp_path):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_mp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "ok").exists()


def _emulated(world, shapes, base, **kw):
    from mojodiffusion_b200.parallel.fused_dp import emulate_ranks
    sets = [[torch.nn.Parameter(b.clone().to("cuda")) for b in base] for _ in range(world)]
    return sets, emulate_ranks(sets, **kw)


def _load_grads(ranks, sets, grads_t):
    for r, rk in enumerate(ranks):
        rk.zero_grad()
        for p, gg in zip(sets[r], grads_t[r]):
            p.grad.copy_(gg.to("cuda"))


def test_optimizer_state_round_trip_gives_identical_next_step():
    """Save (full moments + step), load into fresh ranks, take one more step: parameters are bit-identical to the run that
    never stopped. Also checks set_moments (per-parameter restore, as the LoRA state sidecar uses it) against load_state."""
    from mojodiffusion_b200.ops import native
    from mojodiffusion_b200.parallel.fused_dp import emulated_step
    world = 2
    shapes = [(16, 3072), (3072, 16), (7,), (1000, 33)]
    g = torch.Generator().manual_seed(3)
    base = [torch.randn(*s, generator=g).bfloat16() for s in shapes]
    grads = [[[torch.randn(*s, generator=g).bfloat16() for s in shapes] for _ in range(world)] for _ in range(3)]
    kw = dict(lr=1e-2, weight_decay=0.01, max_grad_norm=1.0)
    sets_a, ranks_a = _emulated(world, shapes, base, **kw)
    for t in range(2):
        _load_grads(ranks_a, sets_a, grads[t])
        emulated_step(ranks_a)
    torch.cuda.synchronize()
    # what gather_state() returns on real ranks: the shards in rank order
    m_full = torch.cat([r.m for r in ranks_a]).clone()
    v_full = torch.cat([r.v for r in ranks_a]).clone()
    weights = [p.detach().clone() for p in sets_a[0]]
    step = ranks_a[0].step_count
    # resumed run B: load_state; resumed run C: set_moments per parameter
    sets_b, ranks_b = _emulated(world, shapes, weights, **kw)
    sets_c, ranks_c = _emulated(world, shapes, weights, **kw)
    for r in ranks_b:
        r.load_state(m_full, v_full, step)
    for r, ps in zip(ranks_c, sets_c):
        for p, o in zip(ps, r.offsets):
            r.set_moments(p, m_full[o:o + p.numel()].view_as(p), v_full[o:o + p.numel()].view_as(p))
        r.step_count = step
    for sets, ranks in ((sets_a, ranks_a), (sets_b, ranks_b), (sets_c, ranks_c)):
        _load_grads(ranks, sets, grads[2])
        emulated_step(ranks)
    torch.cuda.synchronize()
    native.check_status()
    for pa, pb, pc in zip(sets_a[0], sets_b[1], sets_c[0]):
        assert torch.equal(pa.detach(), pb.detach()) and torch.equal(pa.detach(), pc.detach())
    with pytest.raises(RuntimeError):
        ranks_a[0].moments(sets_a[0][0])          # world > 1 and no gather_state() for this step: refuses instead of communicating


def test_timed_out_reduce_leaves_parameters_untouched():
    """A reduce wait that runs out (rank 1 never announces its gradients: a flag nothing sets) must not be followed by an
    optimizer update on stale sums: parameters and moments stay as they were, the done flag is still published, and the
    host gets TIMEOUT from its next status check. The wait limit is lowered to 5 ms for the test and restored after."""
    from mojodiffusion_b200.ops import native
    world = 2
    shapes = [(64, 512), (33,)]
    g = torch.Generator().manual_seed(5)
    base = [torch.randn(*s, generator=g).bfloat16() for s in shapes]
    sets, ranks = _emulated(world, shapes, base, lr=1e-1, weight_decay=0.0, max_grad_norm=0.0)
    for r, rk in enumerate(ranks):
        rk.zero_grad()
        for p in sets[r]:
            p.grad.fill_(1.0)
    native.check_status(ranks[0].red)
    before = ranks[0].flat_params.clone()
    torch.ops.mdb200.set_wait_limit_ns(5_000_000)
    try:
        r0 = ranks[0]
        r0.phase_ready()            # rank 1 never calls phase_ready: its READY flag stays at the old epoch
        r0.phase_reduce()           # -> wait runs out, `red` is not written
        r0.phase_publish()          # -> publishes NaN instead of a partial norm
        r0.phase_update()           # -> skips the update (own status not OK), still publishes DONE
        torch.cuda.synchronize()
        assert torch.equal(r0.flat_params, before), "parameters changed after a timed-out reduce"
        assert float(r0.m.abs().max()) == 0.0 and float(r0.v.abs().max()) == 0.0
        assert int(ranks[1].flags[2 * 8 + 0]) == r0.epoch, "done flag was not published to the peer"
        assert torch.isnan(ranks[1].scalars[0]), "peer should see NaN as this rank's partial norm"
        with pytest.raises(RuntimeError) as e:
            r0.check()
        assert "TIMEOUT" in str(e.value) and "where=201" in str(e.value)
    finally:
        torch.ops.mdb200.set_wait_limit_ns(1_000_000_000)
    native.check_status(ranks[0].red)
