"""CPU tests: IO round trips, schedules, reference-op identities, tiny MMDiT LoRA training, checkpoint layouts."""
import json
import math
import os
import struct

import pytest
import torch

import mojodiffusion_b200.ops as O
from mojodiffusion_b200.io import SafeTensors, ShardedSafeTensors, load_safetensors, save_safetensors, save_sharded
from mojodiffusion_b200.models.mmdit import MMDiT, pack_latents, tiny_mmdit_config, unpack_latents
from mojodiffusion_b200.ops import reference as ref
from mojodiffusion_b200.sampling import flow_match as fm
from mojodiffusion_b200.training import lora as L
from mojodiffusion_b200.training.optim import FusedAdamW
from mojodiffusion_b200.training.trainer import FlowMatchTrainer


def test_safetensors_roundtrip_byte_exact(tmp_path):
    t = {
        "a.weight": torch.randn(4, 6).bfloat16(),
        "b": torch.arange(10, dtype=torch.int64),
        "c.f8": torch.randn(8, 16).to(torch.float8_e4m3fn),
        "scalar": torch.tensor(3.0, dtype=torch.bfloat16),
        "u8": torch.arange(7, dtype=torch.uint8),
    }
    p = tmp_path / "x.safetensors"
    save_safetensors(p, t, {"format": "pt"})
    raw = p.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8:8 + hlen])
    assert list(hdr.keys()) == ["__metadata__", "a.weight", "b", "c.f8", "scalar", "u8"]  # insertion order
    assert b" " not in raw[8:8 + hlen]  # compact header
    assert hdr["scalar"]["shape"] == [] and hdr["c.f8"]["dtype"] == "F8_E4M3"
    st = SafeTensors(p)
    for k, v in t.items():
        got = st.tensor(k)
        assert got.dtype == v.dtype and got.shape == v.shape
        assert torch.equal(got.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else got,
                           v.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else v)
    # rewrite what we read: byte identical file
    p2 = tmp_path / "y.safetensors"
    save_safetensors(p2, {k: st.tensor(k) for k in st.keys()}, st.metadata)
    assert p2.read_bytes() == raw
    st.prefetch_tensor("a.weight")


def test_safetensors_rejects_truncated(tmp_path):
    p = tmp_path / "x.safetensors"
    save_safetensors(p, {"w": torch.randn(64, 64)})
    data = p.read_bytes()
    (tmp_path / "t.safetensors").write_bytes(data[:-100])
    with pytest.raises(ValueError):
        SafeTensors(tmp_path / "t.safetensors")


def test_sharded_index(tmp_path):
    tensors = {f"blocks.{i}.w": torch.randn(32, 32) for i in range(6)}
    idx = save_sharded(tmp_path / "ck", tensors, max_shard_bytes=3 * 32 * 32 * 4)
    sh = ShardedSafeTensors(idx)
    assert sorted(sh.keys()) == sorted(tensors.keys())
    assert len(set(sh.weight_map.values())) == 2
    assert torch.equal(sh.tensor_view("blocks.4.w"), tensors["blocks.4.w"])
    sh2 = ShardedSafeTensors(tmp_path / "ck")  # directory form
    assert torch.equal(sh2.tensor_view("blocks.0.w"), tensors["blocks.0.w"])
    assert sh2.keys_with_prefix("blocks.1.") == ["blocks.1.w"]


def test_flux_schedule_constants():
    s = fm.flux1_sigmas(28, 4096)
    assert len(s) == 29 and s[0] == 1.0 and s[-1] == 0.0
    assert all(a > b for a, b in zip(s, s[1:]))
    mu = fm.flux1_mu(4096)
    assert abs(mu - 1.15) < 1e-12 and abs(fm.flux1_mu(256) - 0.5) < 1e-12
    t = 1 - 1 / 28
    assert abs(s[1] - math.exp(mu) / (math.exp(mu) + (1 / t - 1))) < 1e-12
    z = fm.shifted_sigmas(4, 3.0)
    assert z[0] == 1.0 and z[-1] == 0.0 and abs(z[2] - 3 * 0.5 / (1 + 2 * 0.5)) < 1e-12
    q = fm.qwen_image_sigmas(20, 4096)
    assert len(q) == 21 and abs(q[0] - 1.0) < 1e-9 and abs(q[-2] - 0.02) < 1e-9 and q[-1] == 0.0
    lq = fm.ltx2_linear_quadratic_sigmas(40)
    assert len(lq) == 41 and lq[0] == 1.0 and abs(lq[-1]) < 1e-12 and all(a >= b for a, b in zip(lq, lq[1:]))
    assert abs(fm.flux2_klein_mu(5000, 20) - (0.00016927 * 5000 + 0.45666666)) < 1e-12


def test_pack_unpack_latents():
    z = torch.randn(2, 16, 8, 12)
    x = pack_latents(z)
    assert x.shape == (2, 24, 64)
    # per-token order (c, ph, pw)
    assert torch.equal(x[0, 0].reshape(16, 2, 2), z[0, :, 0:2, 0:2])
    assert torch.equal(unpack_latents(x, 4, 6), z)


def test_rope_is_rotation_and_halfsplit_matches_interleaved_permutation():
    S, H, Dh = 9, 2, 16
    pos = torch.stack([torch.zeros(S), torch.arange(S).float(), torch.arange(S).float() * 2], 1)
    cos, sin = ref.rope_table(pos, (4, 6, 6), 10000.0)
    x = torch.randn(1, S, H, Dh)
    y = ref.apply_rope(x, cos, sin, True)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    back = ref.apply_rope(y, cos, -sin, True)
    assert torch.allclose(back, x, atol=1e-5)
    # half-split result equals interleaved on the permuted vector
    perm = torch.cat([torch.arange(0, Dh, 2), torch.arange(1, Dh, 2)])
    y2 = ref.apply_rope(x[..., perm], cos, sin, False)
    assert torch.allclose(y2, y[..., perm], atol=1e-5)
    assert torch.allclose(cos[0], torch.ones(8)) and torch.allclose(sin[0], torch.zeros(8))


def _tiny(seed=0, dtype=torch.float32):
    return MMDiT(tiny_mmdit_config(), dtype=dtype).init_weights(seed)


def _batch(B=2, seed=1):
    g = torch.Generator().manual_seed(seed)
    x0 = pack_latents(torch.randn(B, 16, 32, 32, generator=g))
    return x0, torch.randn(B, 64, 256, generator=g), torch.randn(B, 256, generator=g)


def test_tiny_mmdit_forward_shapes_and_batch_consistency():
    m = _tiny()
    x0, txt, y = _batch(2)
    t = torch.tensor([0.3, 0.7])
    with torch.no_grad():
        out = m(x0, txt, t, y, hw=(16, 16))
        one = m(x0[1:], txt[1:], t[1:], y[1:], hw=(16, 16))
    assert out.shape == (2, 256, 64)
    assert torch.allclose(out[1:], one, atol=1e-4)


def test_lora_zero_init_is_identity_and_keys_match_layout(tmp_path):
    m = _tiny()
    x0, txt, y = _batch(1)
    t = torch.tensor([0.5])
    with torch.no_grad():
        base = m(x0, txt, t, y, hw=(16, 16))
    slots = L.inject_flux_lora(m, rank=4, alpha=4)
    with torch.no_grad():
        same = m(x0, txt, t, y, hw=(16, 16))
    assert torch.allclose(base, same, atol=1e-5)
    assert [s.key for s in slots] == L.flux_lora_prefixes(2, 2)
    p = tmp_path / "lora.safetensors"
    L.save_lora(p, slots)
    st = SafeTensors(p)
    want = []
    for k in L.flux_lora_prefixes(2, 2):
        want += [f"{k}.alpha", f"{k}.lora_down.weight", f"{k}.lora_up.weight"]
    assert st.keys() == want
    assert st.tensor_info(want[0]).shape == () and st.tensor_info(want[1]).dtype == "BF16"
    assert st.tensor_info("lora_transformer_single_transformer_blocks_0_proj_out.lora_down.weight").shape == (4, 256 + 1024)
    assert st.tensor_info("lora_transformer_transformer_blocks_1_attn_to_k.lora_up.weight").shape == (256, 4)


def test_lora_training_reduces_loss_and_resume_roundtrip(tmp_path):
    torch.manual_seed(0)
    m = _tiny()
    slots = L.inject_flux_lora(m, rank=4, alpha=4)
    params = L.lora_parameters(slots)
    opt = FusedAdamW(params, lr=1e-2, weight_decay=0.01, max_grad_norm=1.0)
    tr = FlowMatchTrainer(m, params, opt)
    x0, txt, y = _batch(2)
    sigma = torch.tensor([0.4, 0.8])
    noise = torch.randn(x0.shape, generator=torch.Generator().manual_seed(5))
    losses = [float(tr.step(x0, txt, y, sigma=sigma, noise=noise, hw=(16, 16))) for _ in range(12)]
    assert all(math.isfinite(l) for l in losses)
    assert losses[-1] < losses[0] - 0.01 and all(b < a for a, b in zip(losses, losses[1:])), losses
    assert all(float(s.up.abs().sum()) > 0 for s in slots)
    # sidecar resume reproduces the next step exactly
    L.save_lora_state_sidecar(tmp_path / "l.state.safetensors", slots, opt, tr.step_index)
    nxt = float(tr.step(x0, txt, y, sigma=sigma, noise=noise, hw=(16, 16)))
    after = [p.detach().clone() for p in params]
    m2 = _tiny()
    slots2 = L.inject_flux_lora(m2, rank=4, alpha=4)
    params2 = L.lora_parameters(slots2)
    opt2 = FusedAdamW(params2, lr=1e-2, weight_decay=0.01, max_grad_norm=1.0)
    step = L.load_lora_state_sidecar(tmp_path / "l.state.safetensors", slots2, opt2)
    assert step == 12
    tr2 = FlowMatchTrainer(m2, params2, opt2)
    nxt2 = float(tr2.step(x0, txt, y, sigma=sigma, noise=noise, hw=(16, 16)))
    # adapters were stored in bf16: compare loosely on the loss, tightly on the moments' effect
    assert abs(nxt - nxt2) < 5e-3 * abs(nxt)
    st = SafeTensors(tmp_path / "l.state.safetensors")
    k0 = slots[0].key
    assert st.tensor_info(f"{k0}.lora_A.adam_m").dtype == "F32" and st.tensor_info(f"{k0}.lora_B.weight").dtype == "BF16"


def test_lora_merge_equals_overlay():
    m = _tiny()
    slots = L.inject_flux_lora(m, rank=4, alpha=8)
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():
        for s in slots:
            s.up.copy_(torch.randn(s.up.shape, generator=g) * 0.05)
    x0, txt, y = _batch(1)
    t = torch.tensor([0.5])
    with torch.no_grad():
        overlay = m(x0, txt, t, y, hw=(16, 16))
        L.merge_lora_into_weights(m)
        merged = m(x0, txt, t, y, hw=(16, 16))
    assert not L.collect_slots(m)
    assert torch.allclose(overlay, merged, atol=2e-4, rtol=1e-3)


def test_adamw_reference_matches_torch():
    p = torch.nn.Parameter(torch.randn(50, 7))
    r = torch.nn.Parameter(p.detach().clone())
    opt = FusedAdamW([p], lr=1e-2, weight_decay=0.05)
    topt = torch.optim.AdamW([r], lr=1e-2, weight_decay=0.05)
    for i in range(4):
        g = torch.randn(50, 7, generator=torch.Generator().manual_seed(i))
        p.grad, r.grad = g.clone(), g.clone()
        opt.step()
        topt.step()
    assert torch.allclose(p, r, atol=1e-6)


def test_euler_sampler_integrates_linear_field():
    # v = -x0 constant field: x(0) = x(1) + (0 - 1) * v
    x = torch.randn(1, 10, 4)
    v = torch.randn(1, 10, 4)
    out = fm.euler_flow_sample(lambda xb, s: v, x.clone(), fm.shifted_sigmas(7, 2.0))
    assert torch.allclose(out, x - v, atol=1e-5)
    out2 = fm.euler_flow_sample(lambda xb, s: v, x.clone(), fm.shifted_sigmas(7, 2.0), uncond_fn=lambda xb, s: 0 * v,
                                cfg_scale=3.0, cfg_mode=fm.CFG_TEXTBOOK)
    assert torch.allclose(out2, x - 3.0 * v, atol=1e-5)


def test_tracing_ranges_and_per_rank_metrics(tmp_path):
    """NVTX ranges are off by default, name stage / block / collective when on; per-rank JSONL files aggregate on rank 0."""
    import torch
    from mojodiffusion_b200.models.mmdit import MMDiT, tiny_mmdit_config
    from mojodiffusion_b200.utils import tracing
    cfg = tiny_mmdit_config()
    model = MMDiT(cfg, torch.float32, "cpu").init_weights(0).eval()
    x, txt, y = torch.randn(1, 16, cfg.in_channels), torch.randn(1, 8, cfg.context_dim), torch.randn(1, cfg.vec_dim)
    log = []
    tracing.set_range_log(log)
    try:
        with torch.no_grad():
            model(x, txt, torch.tensor([0.5]), y, torch.tensor([3.5]), hw=(4, 4))
        assert log == []                                          # disabled: nothing recorded
        tracing.enable_nvtx(True)
        with torch.no_grad(), tracing.nvtx_range("stage/denoise/0"):
            model(x, txt, torch.tensor([0.5]), y, torch.tensor([3.5]), hw=(4, 4))
        assert log[0] == "stage/denoise/0" and "block/double/0" in log and f"block/single/{cfg.depth_single - 1}" in log
    finally:
        tracing.enable_nvtx(False)
        tracing.set_range_log(None)
    for r in range(2):
        m = tracing.MetricsLog(str(tmp_path), r)
        for s in range(3):
            m.log(s, loss=1.0 / (s + 1) + r, ms_per_step=10.0 + r)
        m.close()
    agg = tracing.aggregate(str(tmp_path))
    assert sorted(agg) == [0, 1, 2] and agg[0]["ms_per_step"] == {"min": 10.0, "max": 11.0, "mean": 10.5, "ranks": 2}
    assert abs(agg[2]["loss"]["mean"] - (1 / 3 + 0.5)) < 1e-9
