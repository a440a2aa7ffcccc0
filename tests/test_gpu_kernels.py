"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op (non-degenerate random
fills, small edge shapes and the real DiT shapes)."""
import math

import pytest
import torch

import mojodiffusion_b200.ops as O
from mojodiffusion_b200.ops import native, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
if torch.cuda.is_available():
    native.load(True)


def _rand(*shape, scale=1.0, seed=0, dtype=torch.bfloat16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _cos(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-30))


def _check(out, want, cos=0.9995, rel=2e-2, name=""):
    native.check_status(out)
    assert out.shape == want.shape, (name, out.shape, want.shape)
    assert torch.isfinite(out.float()).all(), name
    c = _cos(out, want)
    err = float((out.float() - want.float()).abs().max())
    ref_mag = float(want.float().abs().max()) + 1e-6
    assert c >= cos, f"{name}: cos {c}"
    assert err <= rel * ref_mag + 1e-3, f"{name}: max err {err} vs magnitude {ref_mag}"


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (200, 264, 72), (1, 64, 64), (4608, 3072, 3072), (512, 9216, 3072),
               (333, 1000, 520), (4096, 64, 3072)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_plain(M, N, K):
    x, w = _rand(M, K, seed=1), _rand(N, K, scale=1 / math.sqrt(K), seed=2)
    out = O.linear(x, w)
    _check(out, ref.linear(x, w, out_dtype=torch.float32), name=f"gemm {M}x{N}x{K}")


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_variants(bn):
    M, N, K = 384, 768, 320
    x, w = _rand(M, K, seed=3), _rand(N, K, scale=1 / math.sqrt(K), seed=4)
    out = torch.ops.mdb200.gemm([x], [w], None, None, None, 1, 0, 0, 0, None, False, False, False, None, None, 1.0,
                                False, bn, None, [], [], [], [], None, None, 0)
    _check(out, ref.linear(x, w, out_dtype=torch.float32), name=f"bn{bn}")


def test_gemm_epilogues():
    B, S, K, N = 2, 300, 256, 512
    x = _rand(B * S, K, seed=5)
    w = _rand(N, K, scale=1 / math.sqrt(K), seed=6)
    bias, gate, res = _rand(N, seed=7), _rand(B, N, seed=8), _rand(B * S, N, seed=9)
    for act in ("gelu_tanh", "silu", "gelu", None):
        out = O.linear(x, w, bias, act=act, residual=res, gate=gate, rows_per_group=S)
        want = ref.linear(x, w, bias, act, res, gate, S, out_dtype=torch.float32)
        _check(out, want, name=f"epilogue {act}")


def test_gemm_segments_and_lora():
    M, K1, K2, N, r = 520, 384, 1024, 640, 16
    a1, a2 = _rand(M, K1, seed=10), _rand(M, K2, seed=11)
    w = _rand(N, K1 + K2, scale=0.03, seed=12)
    out = O.linear(a1, w[:, :K1], extra=[(a2, w[:, K1:])])
    want = ref.linear(torch.cat((a1, a2), 1), w, out_dtype=torch.float32)
    _check(out, want, name="two K segments")
    A, Bm = _rand(r, K1, scale=0.05, seed=13), _rand(N, r, scale=0.05, seed=14)
    out = O.lora_linear(a1, w[:, :K1].contiguous(), None, A, Bm, 0.5)
    want = a1.float() @ w[:, :K1].float().t() + 0.5 * (a1.float() @ A.float().t()).bfloat16().float() @ Bm.float().t()
    _check(out, want, name="lora fused", rel=3e-2)


def test_gemm_paired_swiglu_geglu():
    M, K, F_ = 300, 256, 384
    x = _rand(M, K, seed=15)
    w = _rand(2 * F_, K, scale=1 / math.sqrt(K), seed=16)
    b = _rand(2 * F_, seed=17)
    for act, second in (("silu", False), ("gelu", True)):
        out = O.linear_glu(x, w, b, act, second)
        _check(out, ref.linear_glu(x, w, b, act, second, out_dtype=torch.float32), name=f"glu {act}")


def test_gemm_backward_majors():
    M, N, K = 640, 384, 520
    x = _rand(M, K, seed=18)
    w = _rand(N, K, scale=0.05, seed=19)
    dy = _rand(M, N, seed=20)
    dx = torch.ops.mdb200.gemm([dy], [w], None, None, None, 1, 0, 0, 0, None, False, False, True, None, None, 1.0,
                               False, 0, None, [], [], [], [], None, None, 0)
    _check(dx, dy.float() @ w.float(), name="dx (B MN-major)")
    dw = torch.ops.mdb200.gemm([dy], [x], None, None, None, 1, 0, 0, 0, None, False, True, True, None, None, 1.0,
                               False, 0, None, [], [], [], [], None, None, 0)
    _check(dw, dy.float().t() @ x.float(), name="dW (A,B MN-major)")
    for bn in (64, 128, 256):
        dx = torch.ops.mdb200.gemm([dy], [w], None, None, None, 1, 0, 0, 0, None, False, False, True, None, None, 1.0,
                                   False, bn, None, [], [], [], [], None, None, 0)
        _check(dx, dy.float() @ w.float(), name=f"dx bn{bn}")


def _gemm_bn(As, Bs, bn, **kw):
    from mojodiffusion_b200.ops.functional import _gemm
    return _gemm(As, Bs, bn=bn, **kw)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (300, 384, 200), (4608, 3072, 3072), (1000, 1288, 520)])
def test_gemm_cta_pair_plain(M, N, K):
    """256 x 256 tiles computed by two CTAs (bn=512 forces the CTA-pair kernel), ragged M / N / K included."""
    x, w = _rand(M, K, seed=41), _rand(N, K, scale=1 / math.sqrt(K), seed=42)
    _check(_gemm_bn([x], [w], 512), ref.linear(x, w, out_dtype=torch.float32), name=f"pair {M}x{N}x{K}")


def test_gemm_cta_pair_epilogues_segments_majors():
    B, S, K, N = 2, 300, 256, 512
    x = _rand(B * S, K, seed=43)
    w = _rand(N, K, scale=1 / math.sqrt(K), seed=44)
    bias, gate, res = _rand(N, seed=45), _rand(B, N, seed=46), _rand(B * S, N, seed=47)
    out = _gemm_bn([x], [w], 512, bias=bias, residual=res, gate=gate, rows_per_group=S, act=ref.act_code("gelu_tanh"))
    _check(out, ref.linear(x, w, bias, "gelu_tanh", res, gate, S, out_dtype=torch.float32), name="pair epilogue")
    # two K segments into one accumulator
    a2, w2 = _rand(B * S, 128, seed=48), _rand(N, 128, scale=0.05, seed=49)
    out = _gemm_bn([x, a2], [w, w2], 512)
    _check(out, x.float() @ w.float().t() + a2.float() @ w2.float().t(), name="pair two segments")
    # paired (GLU) mode: the second CTA stages the second operand's rows
    F_ = 384
    wg, bg = _rand(2 * F_, K, scale=1 / math.sqrt(K), seed=50), _rand(2 * F_, seed=51)
    out = _gemm_bn([x], [wg], 512, bias=bg, act=ref.act_code("silu"), pair_offset=F_)
    _check(out, ref.linear_glu(x, wg, bg, "silu", False, out_dtype=torch.float32), name="pair swiglu")
    # gradient layouts: dx = dy W (B MN-major), dW = dy^T x (both MN-major), fp32 output
    M, Nn, Kk = 640, 384, 520
    xx, ww, dy = _rand(M, Kk, seed=52), _rand(Nn, Kk, scale=0.05, seed=53), _rand(M, Nn, seed=54)
    _check(_gemm_bn([dy], [ww], 512, b_mn=True), dy.float() @ ww.float(), name="pair dx")
    _check(_gemm_bn([dy], [xx], 512, a_mn=True, b_mn=True), dy.float().t() @ xx.float(), name="pair dW")
    _check(_gemm_bn([dy], [xx], 512, a_mn=True, b_mn=True, out_fp32=True), dy.float().t() @ xx.float(), name="pair dW fp32")


def test_linear_autograd_matches_torch():
    M, N, K, r = 256, 320, 192, 8
    x = _rand(M, K, seed=21).requires_grad_(True)
    w = _rand(N, K, scale=0.05, seed=22).requires_grad_(True)
    b = _rand(N, seed=23).requires_grad_(True)
    y = O.linear(x, w, b, act="gelu_tanh")
    y.float().square().mean().backward()
    xr, wr, br = [t.detach().float().requires_grad_(True) for t in (x, w, b)]
    torch.nn.functional.gelu(xr @ wr.t() + br, approximate="tanh").square().mean().backward()
    _check(x.grad, xr.grad, cos=0.995, rel=5e-2, name="dx")
    _check(w.grad, wr.grad, cos=0.995, rel=5e-2, name="dw")
    _check(b.grad, br.grad, cos=0.995, rel=5e-2, name="db")
    A = _rand(r, K, scale=0.1, seed=24).requires_grad_(True)
    Bm = _rand(N, r, scale=0.1, seed=25).requires_grad_(True)
    x2 = x.detach().clone().requires_grad_(True)
    y = O.lora_linear(x2, w.detach(), None, A, Bm, 2.0)
    y.float().square().mean().backward()
    xr, Ar, Br = [t.detach().float().requires_grad_(True) for t in (x2, A, Bm)]
    (xr @ w.detach().float().t() + 2.0 * (xr @ Ar.t()) @ Br.t()).square().mean().backward()
    _check(x2.grad, xr.grad, cos=0.995, rel=5e-2, name="lora dx")
    _check(A.grad, Ar.grad, cos=0.99, rel=8e-2, name="lora dA")
    _check(Bm.grad, Br.grad, cos=0.99, rel=8e-2, name="lora dB")


def test_gemm_fp8():
    M, N, K = 300, 512, 1024
    x = _rand(M, K, seed=26)
    w = _rand(N, K, scale=0.05, seed=27)
    wq, ws = O.fp8_quant_rows(w)
    out = O.fp8_linear(x, wq, ws)
    xq, xs = ref.fp8_quant_rows(x)
    want = (xq.float() * xs[:, None]) @ (wq.float() * ws[:, None]).t()
    _check(out, want, name="fp8 gemm")
    _check(out, x.float() @ w.float().t(), cos=0.995, rel=0.1, name="fp8 vs bf16 math")
    _check(O.fp8_dequant(wq, ws), w.float(), cos=0.998, rel=0.08, name="fp8 dequant")


ATT_SHAPES = [(1, 256, 256, 2, 128), (2, 300, 300, 3, 128), (1, 128, 77, 4, 64), (1, 1000, 520, 2, 64),
              (1, 4608, 4608, 4, 128), (2, 640, 256, 2, 128)]


@pytest.mark.parametrize("B,Sq,Skv,H,Dh", ATT_SHAPES)
def test_attention_fwd(B, Sq, Skv, H, Dh):
    q, k, v = _rand(B, Sq, H, Dh, seed=30), _rand(B, Skv, H, Dh, seed=31), _rand(B, Skv, H, Dh, seed=32)
    out = O.attention(q, k, v)
    _check(out, ref.attention(q, k, v).float(), cos=0.999, rel=3e-2, name=f"attn {B},{Sq},{Skv},{H},{Dh}")


def test_attention_strided_and_masked():
    B, S, H, Dh = 2, 520, 3, 128
    qkv = _rand(B, S, 3 * H * Dh, seed=33)
    D = H * Dh
    q, k, v = [qkv[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3)]
    out = O.attention(q, k, v)
    _check(out, ref.attention(q, k, v).float(), cos=0.999, rel=3e-2, name="strided qkv")
    kv_len = torch.tensor([200, 520], dtype=torch.int32, device=DEV)
    out = O.attention(q, k, v, kv_len=kv_len)
    _check(out, ref.attention(q, k, v, kv_len=kv_len).float(), cos=0.999, rel=3e-2, name="kv_len mask")


@pytest.mark.parametrize("fp4", [True, False])
def test_mx_quant_dequant_kernels_match_reference_bit_for_bit(fp4):
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(4096, 96, generator=g) * torch.logspace(-6, 6, 4096)[:, None]).to(DEV).bfloat16()
    x[7, :32] = 0
    q, s = O.mx_quant(x, fp4)
    qr, sr = ref.mx_quant(x, fp4)
    assert torch.equal(s, sr)
    assert torch.equal(q, qr)
    y = O.mx_dequant(q, s, fp4)
    assert torch.equal(y, ref.mx_dequant(q, s, fp4))
    rnd = torch.randint(0, 256, (1000, 16 if fp4 else 32), dtype=torch.uint8, generator=g).to(DEV)
    if not fp4:
        rnd = torch.where((rnd & 0x7F) == 0x7F, torch.zeros_like(rnd), rnd)          # no NaN encodings
    sc = torch.randint(1, 255, (1000,), dtype=torch.uint8, generator=g).to(DEV)
    a, b = O.mx_dequant(rnd, sc, fp4).float(), ref.mx_dequant(rnd, sc, fp4).float()
    assert torch.equal(torch.nan_to_num(a, posinf=9e38, neginf=-9e38), torch.nan_to_num(b, posinf=9e38, neginf=-9e38))


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 520, 384), (4608, 3072, 3072), (1000, 264, 1024), (64, 8, 256)])
def test_gemm_mxfp8_block_scaled(M, N, K):
    """Hardware block-scaled fp8 GEMM against the fp32 product of the dequantised operands (same quantised bytes and scale
    bytes on both sides, so only the accumulation order differs), and the quantiser against its reference bit for bit."""
    g = torch.Generator().manual_seed(M + N + K)
    x = (torch.randn(M, K, generator=g) * torch.logspace(-2, 2, M)[:, None]).to(DEV).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05 * torch.logspace(-1, 1, K)[None, :]).to(DEV).bfloat16()
    bias = torch.randn(N, generator=g).to(DEV).bfloat16()
    xq, xs = O.mxfp8_quant_rows(x, 128)
    wq, ws = O.mxfp8_quant_rows(w, 256)
    xq_r, xs_r = ref.mxfp8_quant_rows(x, 128)
    assert torch.equal(xq, xq_r) and torch.equal(xs, xs_r)
    y = O.gemm_mxfp8(xq, xs, wq, ws, bias)
    want = ref.gemm_mxfp8(xq, xs, wq, ws, bias)
    _check(y, want.float(), cos=0.99999, rel=1e-2, name=f"mxfp8 gemm {M}x{N}x{K}")
    full = x.float() @ w.float().t() + bias.float()
    _check(y, full, cos=0.998, rel=0.1, name="mxfp8 vs bf16 math")


def test_attention_late_large_maximum_is_exact():
    """The exponent reference of a key tile is the row maximum of the EARLIER tiles; rows whose scores jump far above it
    (here by more than 60 nats, several such keys of different height in one tile) take the redo path."""
    B, S, H, Dh = 1, 1024, 2, 128
    q, k, v = _rand(B, S, H, Dh, seed=50), _rand(B, S, H, Dh, seed=51), _rand(B, S, H, Dh, seed=52)
    qn = q.float() / q.float().norm(dim=-1, keepdim=True)
    k = k.clone()
    for key, row, gain in ((700, 5, 9000.0), (710, 5, 8900.0), (705, 300, 12000.0), (900, 640, 20000.0), (130, 64, 7000.0)):
        k[0, key] = (qn[0, row] * gain / math.sqrt(Dh)).to(torch.bfloat16)      # logit of (row, key) ~ gain / Dh * |q|
    out, lse = torch.ops.mdb200.attention_fwd(q, k, v, 1 / math.sqrt(Dh), None, True, None, [], [], [])
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    want, lse_ref = ref.attention(q, k, v, return_lse=True)
    _check(out, want.float(), cos=0.999, rel=3e-2, name="late maximum")
    _check(lse, lse_ref, cos=0.9999, rel=1e-2, name="late maximum lse")
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(Dh)
    first = s[..., :128].amax(-1)
    assert float((s.amax(-1) - first).max()) > 60.0                            # the case really occurs in this input


def test_attention_lse_and_backward():
    B, S, H, Dh = 1, 384, 2, 128
    q, k, v = [_rand(B, S, H, Dh, seed=40 + i).requires_grad_(True) for i in range(3)]
    o = O.attention(q, k, v)
    o.float().square().mean().backward()
    qr, kr, vr = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref.attention(qr, kr, vr).square().mean().backward()
    _check(q.grad, qr.grad, cos=0.99, rel=8e-2, name="dq")
    _check(k.grad, kr.grad, cos=0.99, rel=8e-2, name="dk")
    _check(v.grad, vr.grad, cos=0.99, rel=8e-2, name="dv")
    _, lse = torch.ops.mdb200.attention_fwd(q.detach(), k.detach(), v.detach(), 1 / math.sqrt(Dh), None, True, None, [], [], [])
    _, lse_ref = ref.attention(q.detach(), k.detach(), v.detach(), return_lse=True)
    _check(lse, lse_ref, cos=0.9999, rel=1e-2, name="lse")


def _sinusoid(B, S, H, Dh, phase):
    """Deterministic fill that repeats over no axis: a gradient written to the wrong head, row or column changes the
    result (a random fill with equal statistics per head can hide a head mix-up behind a good cosine)."""
    b = torch.arange(B, device=DEV, dtype=torch.float32).view(B, 1, 1, 1)
    s = torch.arange(S, device=DEV, dtype=torch.float32).view(1, S, 1, 1)
    h = torch.arange(H, device=DEV, dtype=torch.float32).view(1, 1, H, 1)
    d = torch.arange(Dh, device=DEV, dtype=torch.float32).view(1, 1, 1, Dh)
    x = torch.sin(0.37 * s + 1.3 * h + 0.11 * d + 0.7 * b + phase) + 0.5 * torch.cos(0.013 * s * (h + 1) - 0.29 * d + phase)
    return (0.7 * x).to(torch.bfloat16)


ATT_BWD_CASES = [  # B, Sq, Skv, H, Dh, masked
    (1, 1248, 1248, 24, 128, False), (1, 1536, 1536, 30, 128, False), (1, 4608, 4608, 32, 128, False),
    (1, 1536, 1536, 30, 64, False), (2, 1248, 640, 24, 128, False), (1, 640, 1536, 32, 64, False),
    (2, 1536, 1536, 30, 128, True), (2, 1000, 520, 3, 64, True),
]


@pytest.mark.parametrize("B,Sq,Skv,H,Dh,masked", ATT_BWD_CASES)
def test_attention_backward_matrix(B, Sq, Skv, H, Dh, masked):
    """Head counts 24 / 30 / 32 (30 is not a power of two and once produced all-zero dq / dk in the reference), ragged and
    rectangular sequence lengths, key-length masks, both head sizes; gradients against fp32 autograd, per head."""
    q, k, v = _sinusoid(B, Sq, H, Dh, 0.0), _sinusoid(B, Skv, H, Dh, 1.0), _sinusoid(B, Skv, H, Dh, 2.0)
    dout = _sinusoid(B, Sq, H, Dh, 3.0)
    kv_len = torch.tensor([max(1, Skv // 3), Skv][:B], dtype=torch.int32, device=DEV) if masked else None
    scale = 1 / math.sqrt(Dh)
    o, lse = torch.ops.mdb200.attention_fwd(q, k, v, scale, kv_len, True, None, [], [], [])
    dq, dk, dv = torch.ops.mdb200.attention_bwd(q, k, v, o, lse, dout, scale, kv_len, [])
    qr, kr, vr = [t.float().requires_grad_(True) for t in (q, k, v)]
    ref.attention(qr, kr, vr, kv_len=kv_len).backward(dout.float())
    for name, got, want in (("dq", dq, qr.grad), ("dk", dk, kr.grad), ("dv", dv, vr.grad)):
        assert torch.isfinite(got).all(), name
        if masked:                                         # keys past kv_len receive exactly no gradient
            if name in ("dk", "dv"):
                assert float(got[0, int(kv_len[0]):].float().abs().max()) == 0.0, name
        g, w = got.float(), want.float()
        per_head = torch.nn.functional.cosine_similarity(g.permute(2, 0, 1, 3).reshape(H, -1), w.permute(2, 0, 1, 3).reshape(H, -1), dim=1)
        assert float(per_head.min()) > 0.99, f"{name}: worst head cosine {float(per_head.min()):.5f} (head {int(per_head.argmin())})"
        assert float(g.abs().amax(dim=(0, 1, 3)).min()) > 0, f"{name}: a head received no gradient"
        _check(got, want, cos=0.995, rel=8e-2, name=f"{name} {B},{Sq},{Skv},{H},{Dh}")


def test_attention_backward_rejects_bad_arguments():
    q, k, v = _rand(1, 256, 2, 128, seed=1), _rand(1, 256, 2, 128, seed=2), _rand(1, 256, 2, 128, seed=3)
    o, lse = torch.ops.mdb200.attention_fwd(q, k, v, 0.1, None, True, None, [], [], [])
    for bad in (dict(k=k[:, :, :1]), dict(v=v.float()), dict(o=o[:, :128]), dict(dout=o.cpu()), dict(kv_len=torch.zeros(1, dtype=torch.int64, device=DEV))):
        a = dict(q=q, k=k, v=v, o=o, lse=lse, dout=o, kv_len=None)
        a.update(bad)
        with pytest.raises(RuntimeError):
            torch.ops.mdb200.attention_bwd(a["q"], a["k"], a["v"], a["o"], a["lse"], a["dout"], 0.1, a["kv_len"], [])


@pytest.mark.parametrize("rows,D", [(7, 64), (300, 256), (4608, 3072), (33, 4096), (5, 12288)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_modulate(rows, D, rms):
    B = 1 if rows % 3 else 3
    x = _rand(rows, D, seed=50, scale=2.0) + 0.5
    w, b = _rand(D, seed=51), _rand(D, seed=52)
    mod = _rand(B, 2 * D, seed=53, scale=0.3)
    sc, sh = mod[:, :D], mod[:, D:]
    rpg = rows // B
    out = O.norm_modulate(x, w, b, sc, sh, rows_per_group=rpg, eps=1e-6, rms=rms)
    want = ref.norm_modulate(x.float(), w.float(), b.float(), sc.float(), sh.float(), rpg, 1e-6, rms)
    _check(out, want, name="norm fwd")
    xg = x.clone().requires_grad_(True)
    O.norm_modulate(xg, w, None, sc, sh, rows_per_group=rpg, rms=rms).float().square().mean().backward()
    xr = x.float().requires_grad_(True)
    ref.norm_modulate(xr, w.float(), None, sc.float(), sh.float(), rpg, 1e-6, rms).square().mean().backward()
    _check(xg.grad, xr.grad, cos=0.995, rel=5e-2, name="norm dx")


@pytest.mark.parametrize("Dh", [120, 256])
def test_attention_head_widths_outside_the_kernel_use_the_library(Dh):
    """Head widths other than 64 / 128 (Boogu-Image 120, Ideogram-4 256) run instead of failing, with and without a key length."""
    q, k, v = (_rand(2, 70, 3, Dh, seed=70 + i) for i in range(3))
    want = ref.attention(q.float().cpu(), k.float().cpu(), v.float().cpu())
    _check(O.attention(q, k, v), want.to(q.device), cos=0.999, rel=3e-2, name="attention fallback")
    kv_len = torch.tensor([70, 33], dtype=torch.int32, device=q.device)
    want = ref.attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), None, kv_len.cpu())
    _check(O.attention(q, k, v, kv_len=kv_len), want.to(q.device), cos=0.999, rel=3e-2, name="attention fallback masked")
    native.check_status()


@pytest.mark.parametrize("D", [4, 20, 53248])
def test_norm_modulate_widths_outside_the_kernel_use_the_torch_statement(D):
    """Rows that are not a multiple of 8 wide, or wider than 16 384 (Ideogram-4's stacked text features), still normalise."""
    x = _rand(6, D, seed=60, scale=2.0)
    w = _rand(D, seed=61)
    out = O.norm_modulate(x, w, eps=1e-6, rms=True)
    native.check_status()
    _check(out, ref.norm_modulate(x.float(), w.float(), None, None, None, 6, 1e-6, True), name="norm fallback")


@pytest.mark.parametrize("Dh", [64, 128, 256])
@pytest.mark.parametrize("interleaved", [True, False])
def test_qk_norm_rope(Dh, interleaved):
    B, S, H = 2, 77, 3
    D = H * Dh
    qkv = _rand(B, S, 3 * D, seed=60)
    wq, wk = _rand(Dh, seed=61) + 1.0, _rand(Dh, seed=62) + 1.0
    pos = torch.stack([torch.zeros(S + 5), torch.arange(S + 5).float() // 9, torch.arange(S + 5).float() % 9], 1).to(DEV)
    axes = (Dh // 8, 3 * Dh // 8, Dh // 2)
    cos, sin = O.rope_table(pos, axes, 10000.0)
    cr, sr = ref.rope_table(pos, axes, 10000.0)
    _check(cos, cr, cos=0.99999, rel=1e-4, name="rope cos")
    _check(sin, sr, cos=0.99999, rel=1e-4, name="rope sin")
    want = ref.qk_norm_rope(qkv[..., :D].reshape(B, S, H, Dh).float(), qkv[..., D:2 * D].reshape(B, S, H, Dh).float(),
                                         wq.float(), wk.float(), cr[5:], sr[5:], 1e-6, interleaved)
    got = O.qk_norm_rope(qkv.clone(), H, Dh, wq, wk, cos, sin, interleaved=interleaved, pos_offset=5)
    _check(got[..., :D].reshape(B, S, H, Dh), want[0], name="q rope")
    _check(got[..., D:2 * D].reshape(B, S, H, Dh), want[1], name="k rope")
    assert torch.equal(got[..., 2 * D:], qkv[..., 2 * D:])
    # backward through norm + rope
    xg = qkv.clone().requires_grad_(True)
    O.qk_norm_rope(xg, H, Dh, wq, wk, cos, sin, interleaved=interleaved, pos_offset=5).float().square().mean().backward()
    xr = qkv.float().requires_grad_(True)
    q2, k2 = ref.qk_norm_rope(xr[..., :D].reshape(B, S, H, Dh), xr[..., D:2 * D].reshape(B, S, H, Dh), wq.float(),
                              wk.float(), cr[5:], sr[5:], 1e-6, interleaved)
    (torch.cat((q2.reshape(B, S, D), k2.reshape(B, S, D), xr[..., 2 * D:]), -1)).square().mean().backward()
    _check(xg.grad, xr.grad, cos=0.995, rel=5e-2, name="qk_norm_rope dx")


def test_pointwise_family():
    x = _rand(333, 512, seed=70)
    for act in ("gelu_tanh", "gelu", "silu", "sigmoid", "relu", "tanh"):
        _check(O.activation(x, act), ref.activation(x.float(), act), name=act)
        xg = x.clone().requires_grad_(True)
        O.activation(xg, act).float().sum().backward()
        xr = x.float().requires_grad_(True)
        ref.activation(xr, act).sum().backward()
        _check(xg.grad, xr.grad, cos=0.999, rel=3e-2, name=f"{act} grad")
    h = _rand(100, 768, seed=71)
    for act, second in (("silu", False), ("gelu", True)):
        _check(O.glu(h, act, second), ref.glu(h.float(), act, second), name="glu")
        hg = h.clone().requires_grad_(True)
        O.glu(hg, act, second).float().square().sum().backward()
        hr = h.float().requires_grad_(True)
        ref.glu(hr, act, second).square().sum().backward()
        _check(hg.grad, hr.grad, cos=0.999, rel=3e-2, name="glu grad")
    a, y, g = _rand(2, 50, 256, seed=72), _rand(2, 50, 256, seed=73), _rand(2, 256, seed=74)
    _check(O.gate_residual(a, y, g), ref.gate_residual(a.float(), y.float(), g.float(), 50), name="gate_residual")
    _check(O.gate_residual(a, y, g, tanh_gate=True), ref.gate_residual(a.float(), y.float(), g.float(), 50, True),
           name="tanh gate")


def test_sampler_and_flow_kernels():
    n = (3, 1000, 64)
    x = _rand(*n, seed=80, dtype=torch.float32)
    vc, vu = _rand(*n, seed=81), _rand(*n, seed=82)
    for mode in (0, 1, 2):
        xx = x.clone()
        xb = torch.empty_like(xx, dtype=torch.bfloat16)
        O.cfg_euler(xx, vc, vu, dt=-0.03, s=3.5, mode=mode, x_bf16=xb)
        want = ref.cfg_euler(x, vc, vu, -0.03, 3.5, mode)
        _check(xx, want, cos=0.99999, rel=1e-5, name=f"cfg_euler {mode}")
        _check(xb, want, name="bf16 copy")
    x0, eps = _rand(4, 500, 64, seed=83, dtype=torch.float32), _rand(4, 500, 64, seed=84, dtype=torch.float32)
    sig = torch.tensor([0.1, 0.5, 0.9, 1.0], device=DEV)
    xt, tgt = O.flow_match(x0, eps, sig)
    xtr, tgtr = ref.flow_match(x0, eps, sig)
    _check(xt, xtr, name="x_t")
    _check(tgt, tgtr, cos=0.999999, rel=1e-6, name="target")
    pred = _rand(4, 500, 64, seed=85)
    _check(O.mse_loss(pred, tgt).reshape(1), (pred.float() - tgt).pow(2).mean().reshape(1), cos=0.9999, rel=1e-3, name="mse")
    pg = pred.clone().requires_grad_(True)
    O.mse_loss(pg, tgt).backward()
    _check(pg.grad, 2 * (pred.float() - tgt) / pred.numel(), cos=0.999, rel=2e-2, name="mse grad")


def test_randn_distribution_and_determinism():
    a = O.randn((1 << 20,), seed=7, device=DEV)
    b = O.randn((1 << 20,), seed=7, device=DEV)
    c = O.randn((1 << 20,), seed=8, device=DEV)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert abs(float(a.mean())) < 5e-3 and abs(float(a.std()) - 1.0) < 5e-3
    assert abs(float((a < 0).float().mean()) - 0.5) < 5e-3
    assert float(a.abs().max()) < 7.0
    # prefix property: a longer draw with the same seed starts with the shorter one
    d = O.randn((1 << 10,), seed=7, device=DEV)
    assert torch.equal(d, a[: 1 << 10])


def test_fused_adamw_matches_torch():
    from mojodiffusion_b200.training.optim import FusedAdamW
    shapes = [(16, 3072), (3072, 16), (5,), (1000, 33)]
    for pdt in (torch.float32, torch.bfloat16):
        ps = [torch.nn.Parameter(_rand(*s, seed=90 + i, dtype=pdt)) for i, s in enumerate(shapes)]
        rs = [torch.nn.Parameter(p.detach().float().clone()) for p in ps]
        opt = FusedAdamW(ps, lr=1e-2, weight_decay=0.01, max_grad_norm=1.0)
        topt = torch.optim.AdamW(rs, lr=1e-2, weight_decay=0.01, betas=(0.9, 0.999), eps=1e-8)
        for step in range(3):
            for i, (p, r) in enumerate(zip(ps, rs)):
                g = _rand(*p.shape, seed=100 + 10 * step + i, dtype=pdt)
                p.grad = g.clone()
                r.grad = g.float().clone()
            torch.nn.utils.clip_grad_norm_(rs, 1.0)
            opt.step()
            topt.step()
        for p, r in zip(ps, rs):
            _check(p.detach(), r.detach(), cos=0.9999, rel=2e-2 if pdt == torch.bfloat16 else 1e-4, name=f"adamw {pdt}")


def test_adamw_master_weights_and_ema_kernel():
    """Full fine-tune mode: fp32 masters are updated, bf16 model tensors rewritten from them in the same launch; the
    multi-tensor EMA kernel equals shadow = d * shadow + (1 - d) * live."""
    from mojodiffusion_b200.training.ema import EMA
    from mojodiffusion_b200.training.optim import FusedAdamW
    shapes = [(64, 300), (7,), (513, 33)]
    ps = [torch.nn.Parameter(_rand(*s, seed=200 + i, dtype=torch.bfloat16)) for i, s in enumerate(shapes)]
    rs = [torch.nn.Parameter(p.detach().float().clone()) for p in ps]
    opt = FusedAdamW(ps, lr=1e-3, weight_decay=0.01, master_weights=True)
    topt = torch.optim.AdamW(rs, lr=1e-3, weight_decay=0.01)
    ema = EMA(ps, decay=0.9)
    shadow_ref = [p.detach().float().clone() for p in ps]
    for step in range(4):
        for i, (p, r) in enumerate(zip(ps, rs)):
            g = _rand(*p.shape, seed=300 + 10 * step + i, dtype=torch.bfloat16)
            p.grad, r.grad = g.clone(), g.float().clone()
        opt.step()
        topt.step()
        ema.update(step + 1)
        for s, p in zip(shadow_ref, ps):
            s.mul_(0.9).add_(p.detach().float(), alpha=0.1)
    for p, r, m in zip(ps, rs, opt.masters):
        _check(m, r.detach(), cos=0.999999, rel=1e-4, name="fp32 master")
        assert torch.equal(p.detach(), m.bfloat16())             # the model tensor is the rounded master
    for s, sr in zip(ema.shadow, shadow_ref):
        _check(s, sr, cos=0.999999, rel=1e-5, name="ema")


def test_gemm_split_k_skinny_shapes():
    """Skinny GEMMs (LoRA down-projection and its gradients) with the reduction split over idle SMs."""
    from mojodiffusion_b200.ops.functional import _gemm_skinny
    M, K, r, N = 1152, 3072, 16, 3072
    x, A = _rand(M, K, seed=11), _rand(r, K, scale=1 / math.sqrt(K), seed=12)
    _check(_gemm_skinny(x, A), ref.linear(x, A, out_dtype=torch.float32), name="down x@A^T")
    dy, t = _rand(M, N, seed=13), _rand(M, r, seed=14)
    Bs = _rand(N, r, scale=1 / math.sqrt(r), seed=15)
    _check(_gemm_skinny(dy, Bs, b_mn=True), dy.float() @ Bs.float(), name="dt = dy@B")
    _check(_gemm_skinny(t, x, a_mn=True, b_mn=True), t.float().t() @ x.float(), rel=3e-2, name="dA = t^T x")
    _check(_gemm_skinny(dy, t, a_mn=True, b_mn=True, alpha=0.5), 0.5 * (dy.float().t() @ t.float()), rel=3e-2, name="dB = dy^T t")


def test_packed_qkv_attention_matches_composed_ops():
    """The single-node norm/rope + attention path: forward and gradient equal the composed differentiable ops."""
    B, S_txt, S_img, H, Dh = 1, 64, 192, 4, 128
    S, D = S_txt + S_img, H * Dh
    qkv0 = _rand(B, S, 3 * D, seed=21)
    wqa, wka, wqb, wkb = (1.0 + 0.1 * _rand(Dh, seed=22 + i) for i in range(4))
    pos = torch.stack([torch.zeros(S), torch.arange(S).float(), torch.arange(S).float() * 0.5], 1).to(DEV)
    cos, sin = O.rope_table(pos, [16, 56, 56], 10000.0)
    go = _rand(B, S, D, seed=30)
    outs, grads = [], []
    for packed in (True, False):
        qkv = qkv0.clone().requires_grad_(True)
        if packed:
            o = O.qkv_attention(qkv, H, Dh, wqb, wkb, cos, sin, split=S_txt, wq_first=wqa, wk_first=wka)
        else:
            a = O.qk_norm_rope(qkv[:, :S_txt], H, Dh, wqa, wka, cos, sin, pos_offset=0)
            b = O.qk_norm_rope(qkv[:, S_txt:], H, Dh, wqb, wkb, cos, sin, pos_offset=S_txt)
            p = torch.cat((a, b), 1)
            q, k, v = (p[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3))
            o = O.attention(q, k, v).reshape(B, S, D)
        o.backward(go)
        outs.append(o.detach())
        grads.append(qkv.grad.detach())
    assert torch.equal(outs[0], outs[1])
    _check(grads[0], grads[1].float(), cos=0.99999, rel=1e-2, name="packed dqkv")
    h = _rand(B, S, 3 * D + 256, seed=40).requires_grad_(True)
    a, b = O.split_cols(h, 3 * D)
    (a.float().sum() * 2 + b.float().sum() * 3).backward()
    assert a.is_contiguous() and torch.equal(h.grad[..., :3 * D], torch.full_like(a, 2)) and torch.equal(h.grad[..., 3 * D:], torch.full_like(b, 3))


def test_packed_attention_mlp_matches_composed_ops_and_fp32_reference():
    """The middle of a single-stream block as one node (strided column kernels, attention writing into the joint buffer):
    forward and gradient equal the composed ops and agree with the fp32 math of the same expression."""
    B, S, H, Dh, F_ = 2, 256, 4, 128, 1024
    D = H * Dh
    h0 = _rand(B, S, 3 * D + F_, seed=51)
    wq, wk = (1.0 + 0.1 * _rand(Dh, seed=52 + i) for i in range(2))
    pos = torch.stack([torch.zeros(S), torch.arange(S).float(), torch.arange(S).float() * 0.5], 1).to(DEV)
    cos, sin = O.rope_table(pos, [16, 56, 56], 10000.0)
    go = _rand(B, S, D + F_, seed=55)
    outs, grads = [], []
    for packed in (True, False):
        h = h0.clone().requires_grad_(True)
        if packed:
            o = O.packed_attention_mlp(h, H, Dh, wq, wk, cos, sin, act="gelu_tanh")
        else:
            qkv, mlp = O.split_cols(h, 3 * D)
            o = torch.cat((O.qkv_attention(qkv, H, Dh, wq, wk, cos, sin), O.activation(mlp, "gelu_tanh")), -1)
        o.backward(go)
        outs.append(o.detach())
        grads.append(h.grad.detach())
    assert torch.equal(outs[0], outs[1])
    _check(grads[0], grads[1].float(), cos=0.99999, rel=1e-2, name="packed dh")
    # fp32 oracle of the same expression on the reference ops
    hf = h0.float().cpu().requires_grad_(True)
    of = O.packed_attention_mlp(hf, H, Dh, wq.float().cpu(), wk.float().cpu(), cos.cpu(), sin.cpu(), act="gelu_tanh")
    of.backward(go.float().cpu())
    _check(outs[0], of.detach().to(DEV), cos=0.9999, rel=3e-2, name="packed forward vs fp32")
    _check(grads[0], hf.grad.to(DEV), cos=0.999, rel=6e-2, name="packed dh vs fp32")
    # gated (SwiGLU) MLP half: [q | k | v | gate | up] -> [attention | silu(gate) * up]
    hg0 = _rand(B, S, 3 * D + 2 * F_, seed=62)
    res = []
    for packed in (True, False):
        h = hg0.clone().requires_grad_(True)
        if packed:
            o = O.packed_attention_mlp(h, H, Dh, wq, wk, cos, sin, act="silu", gated=False)
        else:
            qkv, mlp = O.split_cols(h, 3 * D)
            o = torch.cat((O.qkv_attention(qkv, H, Dh, wq, wk, cos, sin), O.glu(mlp, "silu", False)), -1)
        o.backward(go)
        res.append((o.detach(), h.grad.detach()))
    assert torch.equal(res[0][0], res[1][0])
    _check(res[0][1], res[1][1].float(), cos=0.99999, rel=1e-2, name="packed gated dh")
    # strided copy / activation kernels against torch on odd row strides
    x = _rand(96, 640, seed=60)
    dst = torch.zeros(96, 512, dtype=torch.bfloat16, device=DEV)
    torch.ops.mdb200.act_strided(x[:, 128:384], None, dst[:, 64:320], 0)
    assert torch.equal(dst[:, 64:320], x[:, 128:384]) and float(dst[:, :64].abs().sum()) == 0 and float(dst[:, 320:].abs().sum()) == 0
    # gate_mul = the gated branch's gradient
    gate = _rand(2, 640, seed=61)
    gm = torch.ops.mdb200.gate_mul(x, gate, 48, False)
    _check(gm, x.float() * gate.float().repeat_interleave(48, 0), rel=1e-2, name="gate_mul")


def test_adamw8bit_kernel_matches_blockwise_reference():
    """The one-kernel 8-bit AdamW (block-wise code-book moments) against the same optimizer stepped on the CPU with the
    tensor-op de-quantise / update / re-quantise sequence."""
    from mojodiffusion_b200.training.optim_extra import AdamW8bit, dequantize_blockwise
    g = torch.Generator().manual_seed(31)
    shapes = [(300, 257), (1000,), (64, 64)]
    ps_cpu = [torch.nn.Parameter(torch.randn(*s, generator=g)) for s in shapes]
    ps_gpu = [torch.nn.Parameter(p.detach().clone().to(DEV)) for p in ps_cpu]
    o_cpu, o_gpu = AdamW8bit(ps_cpu, lr=1e-2, weight_decay=0.05), AdamW8bit(ps_gpu, lr=1e-2, weight_decay=0.05)
    for step in range(4):
        for pc, pg in zip(ps_cpu, ps_gpu):
            gr = torch.randn(pc.shape, generator=g) * (0.5 + step)
            pc.grad, pg.grad = gr.clone(), gr.to(DEV)
        o_cpu.step(grad_scale=0.5)
        o_gpu.step(grad_scale=0.5)
    native.check_status()
    for pc, pg in zip(ps_cpu, ps_gpu):
        _check(pg.detach().cpu(), pc.detach(), cos=0.99999, rel=2e-3, name="param")
        sc, sg = o_cpu.state[id(pc)], o_gpu.state[id(pg)]
        mc = dequantize_blockwise(sc["qm"], sc["am"], o_cpu.code_s, pc.shape, 256)
        mg = dequantize_blockwise(sg["qm"].cpu(), sg["am"].cpu(), o_cpu.code_s, pc.shape, 256)
        assert _cos(mg, mc) > 0.9995
        assert (sg["qm"].cpu() != sc["qm"]).float().mean() < 0.02       # a code may differ by one where rounding ties


def test_bounded_wait_runs_out_and_reports_status():
    """Failure detection on the device: a kernel waits for a peer flag that nothing ever sets. Its wait is bounded (one
    second of wall clock), so it returns, records TIMEOUT with the place and the silent rank in the status word, and the
    host raises from check_status; the context stays usable (a GEMM right after gives the right answer)."""
    import time
    flags = torch.zeros(8 * 8, dtype=torch.int32, device=DEV)              # [slots, ranks]: this rank's arrival flags
    flags[3 * 8 + 0] = 5                                                    # rank 0 arrived at epoch 5, rank 1 never does
    native.check_status(flags)                                             # clean slate
    t0 = time.time()
    torch.ops.mdb200.flag_wait(flags, 3, 2, 5, None)
    with pytest.raises(RuntimeError) as e:
        native.check_status(flags)
    dt = time.time() - t0
    assert "TIMEOUT" in str(e.value) and "where=103" in str(e.value) and "extra=1" in str(e.value)
    assert 0.9 < dt < 5.0, dt                                              # gave up after about a second, not earlier
    native.check_status(flags)                                             # the status word was reset by the read
    x, w = _rand(256, 128, seed=61), _rand(192, 128, scale=0.1, seed=62)
    _check(O.linear(x, w), ref.linear(x, w, out_dtype=torch.float32), name="gemm after a timed-out wait")


def _poisoned(rows, cols, pad_r, pad_c, dtype=torch.bfloat16):
    buf = torch.full((rows + 2 * pad_r, cols + 2 * pad_c), float("nan"), dtype=dtype, device=DEV)
    return buf, buf[pad_r:pad_r + rows, pad_c:pad_c + cols]


@pytest.mark.parametrize("M,N,K", [(200, 264, 72), (333, 1000, 520), (512, 768, 256), (130, 8, 64)])
def test_gemm_writes_exactly_its_output_region(M, N, K):
    """Race / overrun substitute for a memory checker: the output lives inside a NaN-filled buffer with guard rows and
    columns; afterwards no NaN survives inside and every guard element is still NaN (nothing outside the tile was touched,
    ragged edges included, for the direct and the shared-memory-staged epilogue)."""
    x, w = _rand(M, K, seed=71), _rand(N, K, scale=1 / math.sqrt(K), seed=72)
    buf, view = _poisoned(M, N, 3, 8)
    from mojodiffusion_b200.ops.functional import _gemm
    for bn in (0, 256, 512, 128, 64):
        buf.fill_(float("nan"))
        _gemm([x], [w], out=view, bn=bn)
        _check(view, ref.linear(x, w, out_dtype=torch.float32), name=f"poison gemm bn={bn}")
        guard = buf.clone()
        guard[3:3 + M, 8:8 + N] = float("nan")
        assert torch.isnan(guard).all(), f"bn={bn}: the kernel wrote outside its output"


def test_attention_writes_exactly_its_output_region():
    B, Sq, Skv, H, Dh = 1, 300, 200, 2, 128
    q, k, v = _rand(B, Sq, H, Dh, seed=73), _rand(B, Skv, H, Dh, seed=74), _rand(B, Skv, H, Dh, seed=75)
    buf = torch.full((B, Sq + 6, H, Dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = buf[:, 3:3 + Sq]
    torch.ops.mdb200.attention_fwd(q, k, v, 1 / math.sqrt(Dh), None, False, out, [], [], [])
    want = ref.attention(q, k, v, 1 / math.sqrt(Dh))
    _check(out, want, cos=0.999, name="poison attention")
    assert torch.isnan(buf[:, :3]).all() and torch.isnan(buf[:, 3 + Sq:]).all()


# ---- convolution / GroupNorm in training -------------------------------------------------------------------------------
@pytest.mark.parametrize("Cin,Cout,K,stride,offset", [(64, 128, 3, 1, 0), (4, 320, 3, 1, 0), (128, 3, 3, 1, 0), (320, 320, 3, 2, 0),
                                                      (128, 128, 3, 2, 1), (192, 64, 1, 1, 0)])
def test_conv2d_forward_and_gradients_native(Cin, Cout, K, stride, offset):
    """Any channel count and the two stride-2 forms on the implicit-GEMM kernel; input, weight and bias gradients against
    fp32 autograd of torch's convolution."""
    from mojodiffusion_b200.ops import conv as C
    g = torch.Generator().manual_seed(Cin + Cout)
    N, H, W = 2, 24, 20
    x = torch.randn(N, H, W, Cin, generator=g).to(DEV).bfloat16().requires_grad_(True)
    w = (torch.randn(Cout, K, K, Cin, generator=g) * (1.0 / math.sqrt(K * K * Cin))).to(DEV).bfloat16().requires_grad_(True)
    b = torch.randn(Cout, generator=g).to(DEV).bfloat16().requires_grad_(True)
    pad = K // 2
    y = C.conv2d_nhwc(x, w, b, stride, pad, offset=offset)
    xr, wr, br = [t.detach().float().requires_grad_(True) for t in (x, w, b)]
    xin = xr.permute(0, 3, 1, 2)
    if stride == 2 and offset == 1:
        yr = torch.nn.functional.conv2d(torch.nn.functional.pad(xin, (0, 1, 0, 1)), wr.permute(0, 3, 1, 2), br, stride=2, padding=0)
    else:
        yr = torch.nn.functional.conv2d(xin, wr.permute(0, 3, 1, 2), br, stride=stride, padding=pad)
    yr = yr.permute(0, 2, 3, 1)
    assert y.shape == yr.shape
    _check(y, yr, cos=0.9995, rel=3e-2, name="conv fwd")
    dy = torch.randn(y.shape, generator=g).to(DEV)
    y.backward(dy.bfloat16())
    yr.backward(dy.bfloat16().float())
    _check(x.grad, xr.grad, cos=0.999, rel=4e-2, name="conv dx")
    _check(w.grad, wr.grad, cos=0.999, rel=4e-2, name="conv dw")
    _check(b.grad, br.grad, cos=0.999, rel=4e-2, name="conv db")
    with torch.no_grad():
        _check(C.conv2d_nhwc(x.detach(), w.detach(), b.detach(), stride, pad, offset=offset), yr.detach(), cos=0.9995, rel=3e-2, name="conv inference")


@pytest.mark.parametrize("C_,G,act", [(320, 32, "silu"), (128, 32, None), (64, 8, "silu")])
def test_group_norm_backward_kernel(C_, G, act):
    from mojodiffusion_b200.ops import conv as C
    g = torch.Generator().manual_seed(C_)
    x = (torch.randn(2, 12, 10, C_, generator=g) * 2 + 0.5).to(DEV).bfloat16().requires_grad_(True)
    w = (1 + 0.2 * torch.randn(C_, generator=g)).to(DEV).bfloat16().requires_grad_(True)
    b = (0.2 * torch.randn(C_, generator=g)).to(DEV).bfloat16().requires_grad_(True)
    y = C.group_norm_nhwc(x, w, b, G, 1e-5, act)
    xr, wr, br = [t.detach().float().requires_grad_(True) for t in (x, w, b)]
    yr = torch.nn.functional.group_norm(xr.permute(0, 3, 1, 2), G, wr, br, 1e-5)
    yr = (torch.nn.functional.silu(yr) if act else yr).permute(0, 2, 3, 1)
    _check(y, yr, cos=0.9995, rel=3e-2, name="gn fwd")
    dy = torch.randn(y.shape, generator=g).to(DEV).bfloat16()
    y.backward(dy)
    yr.backward(dy.float())
    _check(x.grad, xr.grad, cos=0.999, rel=4e-2, name="gn dx")
    _check(w.grad, wr.grad, cos=0.999, rel=4e-2, name="gn dw")
    _check(b.grad, br.grad, cos=0.999, rel=4e-2, name="gn db")


def test_unet_lora_step_runs_without_library_convolutions(monkeypatch):
    """A LoRA step of the (tiny) UNet: every convolution and GroupNorm, forward and backward, is one of this package's
    kernels; torch's convolution is never entered."""
    from mojodiffusion_b200.models.unet import UNet, tiny_unet_config
    from mojodiffusion_b200.training import lora as L
    calls = {"n": 0}
    orig = torch.nn.functional.conv2d

    def spy(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)
    m = UNet(tiny_unet_config(), torch.bfloat16, DEV).init_weights(0)
    slots = L.inject_sdxl_lora(m, rank=4, alpha=4.0)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 4, 16, 16, generator=g).to(DEV)
    ctx = torch.randn(2, 7, 64, generator=g).to(DEV)
    y = torch.randn(2, 96, generator=g).to(DEV)
    monkeypatch.setattr(torch.nn.functional, "conv2d", spy)
    out = m(x, torch.tensor([10.0, 500.0], device=DEV), ctx, y)
    out.float().square().mean().backward()
    native.check_status(out)
    assert calls["n"] == 0
    assert all(s.up.grad is not None for s in slots) and any(float(s.down.grad.abs().sum()) > 0 or float(s.up.grad.abs().sum()) > 0 for s in slots)


def test_linear_pads_odd_reduction_and_output_widths():
    """Patch embedders with 65 or 132 input values per token and heads with narrow outputs: rows that are not 16-byte
    multiples are zero-padded on the way in and sliced on the way out, with and without autograd."""
    for K, N in ((65, 128), (132, 64), (64, 12), (20, 4)):
        x, w, b = _rand(96, K, seed=K), _rand(N, K, seed=K + 1) * 0.1, _rand(N, seed=K + 2)
        y = O.linear(x, w, b, act="silu")
        _check(y, torch.nn.functional.silu(x.float() @ w.float().t() + b.float()), name=f"linear K={K} N={N}")
        assert y.shape == (96, N) and y.is_contiguous()
        xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        O.linear(xg, wg, b).float().square().sum().backward()
        xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
        (xr @ wr.t() + b.float()).square().sum().backward()
        _check(xg.grad, xr.grad, rel=5e-2, name="dx of padded linear")
        _check(wg.grad, wr.grad, rel=5e-2, name="dw of padded linear")


def test_lion_and_stable_adamw_device_kernels_match_the_torch_statements():
    """Lion and StableAdamW: the multi-tensor device launches against the same optimizers' torch statements on the CPU,
    several steps, fp32 and bf16 parameters, tensors of unequal size."""
    from mojodiffusion_b200.training.optim_extra import Lion, StableAdamW
    for cls, kw in ((Lion, dict(lr=1e-2, weight_decay=0.1)), (StableAdamW, dict(lr=1e-2, weight_decay=0.1))):
        for dt in (torch.float32, torch.bfloat16):
            g = torch.Generator().manual_seed(3)
            shapes = [(300, 70), (5000,), (17,)]
            cpu = [torch.nn.Parameter(torch.randn(s, generator=g).to(dt)) for s in shapes]
            gpu = [torch.nn.Parameter(p.detach().clone().to(DEV)) for p in cpu]
            oc, og = cls(cpu, **kw), cls(gpu, **kw)
            for step in range(4):
                for pc, pg in zip(cpu, gpu):
                    gr = torch.randn(pc.shape, generator=g) * (1.0 + step)
                    pc.grad, pg.grad = gr.to(dt), gr.to(dt).to(DEV)
                oc.step(grad_scale=0.5)
                og.step(grad_scale=0.5)
            torch.cuda.synchronize()
            native.check_status()
            assert getattr(og, "_table", None) is not None, "the device path did not run"
            for pc, pg in zip(cpu, gpu):
                tol = 3e-2 if dt == torch.bfloat16 else 2e-5
                assert (pc.detach().float() - pg.detach().float().cpu()).abs().max() < tol, (cls.__name__, dt)
                assert (oc.m[id(pc)] - og.m[id(pg)].cpu()).abs().max() < 1e-4
