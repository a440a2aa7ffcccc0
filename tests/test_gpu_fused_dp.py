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
