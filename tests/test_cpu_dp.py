"""Data-parallel plumbing on CPU ranks (gloo, world_size 2): a tiny FLUX-style MMDiT LoRA step under DP-2 must
reproduce the single-rank batch-2 trajectory (same loss mean, same adapters after the update)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mojodiffusion_b200.models.mmdit import MMDiT, pack_latents, tiny_mmdit_config
from mojodiffusion_b200.parallel.dp import DataParallelGrads
from mojodiffusion_b200.training import lora as L
from mojodiffusion_b200.training.optim import FusedAdamW
from mojodiffusion_b200.training.trainer import FlowMatchTrainer


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _data():
    g = torch.Generator().manual_seed(11)
    x0 = pack_latents(torch.randn(2, 16, 32, 32, generator=g))
    txt = torch.randn(2, 64, 256, generator=g)
    y = torch.randn(2, 256, generator=g)
    sigma = torch.tensor([0.35, 0.75])
    noise = torch.randn(x0.shape, generator=g)
    return x0, txt, y, sigma, noise


def _make(dp_group=None, use_dp=False):
    m = MMDiT(tiny_mmdit_config(), dtype=torch.float32).init_weights(0)
    slots = L.inject_flux_lora(m, rank=4, alpha=4)
    params = L.lora_parameters(slots)
    opt = FusedAdamW(params, lr=1e-4, betas=(0.9, 0.999), weight_decay=0.01)
    dp = DataParallelGrads(params, dp_group) if use_dp else None
    return m, slots, params, FlowMatchTrainer(m, params, opt, dp)


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    x0, txt, y, sigma, noise = _data()
    m, slots, params, tr = _make(use_dp=True)
    sl = slice(rank, rank + 1)
    losses = []
    for _ in range(3):
        losses.append(tr.step(x0[sl], txt[sl], y[sl], sigma=sigma[sl], noise=noise[sl], hw=(16, 16)))
    lt = torch.stack(losses)
    dist.all_reduce(lt)
    if rank == 0:
        torch.save({"loss": lt / world, "params": [p.detach().clone() for p in params]}, os.path.join(out_dir, "dp.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_dp2_gloo_matches_single_rank_batch2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / "dp.pt")
    x0, txt, y, sigma, noise = _data()
    m, slots, params, tr = _make()
    losses = [tr.step(x0, txt, y, sigma=sigma, noise=noise, hw=(16, 16)) for _ in range(3)]
    want_loss = torch.stack(losses)
    assert torch.allclose(got["loss"], want_loss, rtol=1e-5, atol=1e-6), (got["loss"], want_loss)
    for a, b in zip(got["params"], params):
        assert torch.allclose(a, b.detach(), rtol=1e-4, atol=1e-7)
