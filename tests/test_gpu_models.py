"""Model families on the GPU kernels (bf16) against the same modules evaluated through the pure-torch references in
fp32 on the CPU; convolution / GroupNorm kernels against torch."""
import copy
import math

import pytest
import torch

import mojodiffusion_b200.ops as O
from mojodiffusion_b200.ops import conv as C
from mojodiffusion_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cos(a, b):
    a, b = a.float().flatten().cpu(), b.float().flatten().cpu()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-30))


def _gpu_vs_cpu(make, inputs, cos_min=0.995, **kw):
    m32 = make(torch.float32, "cpu").init_weights(0)
    mg = make(torch.bfloat16, DEV)
    mg.load_state_dict({k: v.to(torch.bfloat16) for k, v in m32.state_dict().items()})
    with torch.no_grad():
        m32.load_state_dict({k: v.float() for k, v in mg.state_dict().items()})   # same bf16-rounded weights
        want = m32(*inputs, **kw)
        got = mg(*[t.to(DEV) for t in inputs], **kw)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.isfinite(got.float()).all()
    c = _cos(got, want)
    assert c >= cos_min, f"cos {c}"
    return got


@pytest.mark.parametrize("cin,cout,k,hw", [(64, 64, 3, (16, 16)), (128, 256, 3, (24, 40)), (256, 128, 1, (9, 13)), (64, 8, 3, (8, 8))])
def test_conv2d_implicit_gemm(cin, cout, k, hw):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, hw[0], hw[1], cin, generator=g).bfloat16().to(DEV)
    w = (torch.randn(cout, k, k, cin, generator=g) / math.sqrt(cin * k * k)).bfloat16().to(DEV)
    b = torch.randn(cout, generator=g).bfloat16().to(DEV)
    res = torch.randn(2, hw[0], hw[1], cout, generator=g).bfloat16().to(DEV)
    with torch.no_grad():
        got = C.conv2d_nhwc(x, w, b, 1, k // 2, "silu", res)
        want = C.conv2d_nhwc_reference(x.float(), w.float(), b.float(), 1, k // 2, "silu", res.float())
    native.check_status(got)
    assert _cos(got, want) > 0.9995 and float((got.float() - want).abs().max()) < 0.06 * float(want.abs().max()) + 1e-2


def test_group_norm_upsample_pool():
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(2, 12, 10, 128, generator=g) * 2 + 0.3).bfloat16().to(DEV)
    w, b = torch.randn(128, generator=g).bfloat16().to(DEV), torch.randn(128, generator=g).bfloat16().to(DEV)
    with torch.no_grad():
        for act in (None, "silu"):
            got = C.group_norm_nhwc(x, w, b, 32, 1e-6, act)
            want = torch.nn.functional.group_norm(x.float().permute(0, 3, 1, 2), 32, w.float(), b.float(), 1e-6)
            want = (torch.nn.functional.silu(want) if act else want).permute(0, 2, 3, 1)
            assert _cos(got, want) > 0.9995
        up = C.upsample_nearest2x_nhwc(x)
        assert torch.equal(up, x.repeat_interleave(2, 1).repeat_interleave(2, 2))
        pool = C.avgpool2x_nhwc(x)
        assert _cos(pool, x.float().reshape(2, 6, 2, 5, 2, 128).mean((2, 4))) > 0.9999
    native.check_status(x)


def test_single_stream_dit():
    from mojodiffusion_b200.models.single_dit import SingleStreamDiT, tiny_single_dit_config
    g = torch.Generator().manual_seed(2)
    inputs = (torch.randn(2, 64, 64, generator=g), torch.randn(2, 16, 128, generator=g), torch.tensor([0.2, 0.9]))
    _gpu_vs_cpu(lambda dt, dev: SingleStreamDiT(tiny_single_dit_config(), dt, dev), inputs, hw=(8, 8))


def test_flux2_klein_dit_forward_and_lora_grads():
    """FLUX.2 Klein-shaped MMDiT: inference path (GLU-epilogue GEMMs, packed attention) against the fp32 CPU modules, and
    the LoRA gradients of the training path against the CPU autograd result."""
    from mojodiffusion_b200.models.flux2 import Flux2DiT, tiny_flux2_config
    from mojodiffusion_b200.training import lora as L
    g = torch.Generator().manual_seed(5)
    cfg = tiny_flux2_config()
    inputs = (torch.randn(2, 64, cfg.in_channels, generator=g), torch.randn(2, 16, cfg.context_dim, generator=g), torch.tensor([0.2, 0.9]))
    _gpu_vs_cpu(lambda dt, dev: Flux2DiT(cfg, dt, dev), inputs, hw=(8, 8))
    grads = []
    for dt, dev in ((torch.float32, "cpu"), (torch.bfloat16, DEV)):
        m = Flux2DiT(cfg, torch.float32, "cpu").init_weights(0)
        slots = L.inject_lora_by_name(m, {n: n for n in m.lora_target_names()}, rank=8, alpha=8.0)
        gg = torch.Generator().manual_seed(6)
        for s_ in slots:
            s_.up.data.copy_(torch.randn(s_.up.shape, generator=gg) * 0.05)
        m = m.to(dev, dt)
        m.gradient_checkpointing = True
        m.train()
        out = m(*[t.to(dev) for t in inputs], hw=(8, 8))
        out.float().pow(2).mean().backward()
        grads.append(torch.cat([p.grad.float().flatten().cpu() for p in L.lora_parameters(L.collect_slots(m))]))
    native.check_status()
    assert _cos(grads[1], grads[0]) > 0.98, _cos(grads[1], grads[0])


def test_qwen_image_dit_with_text_mask():
    from mojodiffusion_b200.models.qwen_image import QwenImageDiT, tiny_qwen_image_config
    g = torch.Generator().manual_seed(3)
    inputs = (torch.randn(2, 64, 64, generator=g), torch.randn(2, 24, 128, generator=g), torch.tensor([0.3, 0.7]))
    m32 = QwenImageDiT(tiny_qwen_image_config(), torch.float32, "cpu").init_weights(0)
    mg = QwenImageDiT(tiny_qwen_image_config(), torch.bfloat16, DEV)
    mg.load_state_dict({k: v.bfloat16() for k, v in m32.state_dict().items()})
    m32.load_state_dict({k: v.float() for k, v in mg.state_dict().items()})
    tl = torch.tensor([24, 9], dtype=torch.int32)
    with torch.no_grad():
        want = m32(*inputs, hw=(8, 8), txt_len=tl)
        got = mg(*[t.to(DEV) for t in inputs], hw=(8, 8), txt_len=tl.to(DEV))
    native.check_status(got)
    assert _cos(got, want) > 0.995


def test_video_dit_bf16_and_fp8():
    from mojodiffusion_b200.models.video_dit import VideoDiT, tiny_video_dit_config
    g = torch.Generator().manual_seed(4)
    inputs = (torch.randn(2, 2 * 4 * 8, 32, generator=g), torch.randn(2, 10, 128, generator=g), torch.tensor([0.3, 0.6]))
    got = _gpu_vs_cpu(lambda dt, dev: VideoDiT(tiny_video_dit_config(), dt, dev), inputs, grid=(2, 4, 8))
    m = VideoDiT(tiny_video_dit_config(), torch.bfloat16, DEV).init_weights(0)
    with torch.no_grad():
        ref = m(*[t.to(DEV) for t in inputs], grid=(2, 4, 8))
        q = copy.deepcopy(m).to_fp8()
        out = q(*[t.to(DEV) for t in inputs], grid=(2, 4, 8))
        qb = copy.deepcopy(m).to_fp8(block_scaled=True)              # MXFP8 weights and activations, hardware block scaling
        out_b = qb(*[t.to(DEV) for t in inputs], grid=(2, 4, 8))
    native.check_status(out)
    assert _cos(out, ref) > 0.99
    assert _cos(out_b, ref) > 0.99 and type(qb.transformer_blocks[0].ff.net["2"]).__name__ == "MXFP8Linear"


def test_unet_and_vae():
    from mojodiffusion_b200.models.unet import UNet, tiny_unet_config
    from mojodiffusion_b200.models.vae import AutoencoderKL, tiny_vae_config
    g = torch.Generator().manual_seed(5)
    inputs = (torch.randn(2, 4, 16, 16, generator=g), torch.tensor([10.0, 900.0]), torch.randn(2, 7, 64, generator=g),
              torch.randn(2, 96, generator=g))
    _gpu_vs_cpu(lambda dt, dev: UNet(tiny_unet_config(), dt, dev), inputs, cos_min=0.99)
    v32 = AutoencoderKL(tiny_vae_config(), torch.float32, "cpu").init_weights(0)
    vg = AutoencoderKL(tiny_vae_config(), torch.bfloat16, DEV)
    vg.load_state_dict({k: v.bfloat16() for k, v in v32.state_dict().items()})
    v32.load_state_dict({k: v.float() for k, v in vg.state_dict().items()})
    z = torch.randn(1, 4, 12, 12, generator=g)
    with torch.no_grad():
        want = v32.decode(z)
        got = vg.decode(z.to(DEV))
        enc = vg.encode(torch.randn(1, 3, 32, 32, generator=g).to(DEV), sample=False)
        tiled = vg.tiled_decode(torch.randn(1, 4, 24, 24, generator=g).to(DEV), tile=16, overlap=8)
    native.check_status(got)
    assert _cos(got, want) > 0.99 and enc.shape == (1, 4, 16, 16) and tiled.shape == (1, 3, 48, 48)
    assert torch.isfinite(tiled.float()).all()


def test_cuda_graph_replay_is_bit_exact():
    from mojodiffusion_b200.models.mmdit import MMDiT, tiny_mmdit_config
    from mojodiffusion_b200.utils.cuda_graph import graphs_equal_eager
    m = MMDiT(tiny_mmdit_config(), torch.bfloat16, DEV).init_weights(0)
    g = torch.Generator().manual_seed(6)
    img = torch.randn(1, 256, 64, generator=g).bfloat16().to(DEV)
    txt = torch.randn(1, 64, 256, generator=g).bfloat16().to(DEV)
    y = torch.randn(1, 256, generator=g).bfloat16().to(DEV)
    t = torch.tensor([0.5], device=DEV)
    ids = MMDiT.make_ids(16, 16, 64, DEV)
    same, err = graphs_equal_eager(lambda a, b, c, d: m(a, b, c, d, ids=ids), [img, txt, t, y])
    native.check_status(img)
    assert same, err


def test_sharded_model_full_finetune_step_matches_unsharded():
    """Model-level FSDP wrapping on one rank: every large Linear of a tiny Qwen-Image-shaped MMDiT becomes a ShardedLinear
    (fp32 master + AdamW moments per shard, activation / gated residual after the projection); two full-finetune steps
    give the losses and weights of the same model trained unsharded with fp32-master AdamW."""
    from mojodiffusion_b200.models.layers import Linear
    from mojodiffusion_b200.models.qwen_image import QwenImageDiT, tiny_qwen_image_config
    from mojodiffusion_b200.parallel.fsdp import FSDPContext, ShardedLinear, shard_model
    from mojodiffusion_b200.training.optim import FusedAdamW
    cfg = tiny_qwen_image_config()
    g = torch.Generator().manual_seed(8)
    x0 = torch.randn(1, 64, cfg.in_channels, generator=g).to(DEV)
    eps = torch.randn(1, 64, cfg.in_channels, generator=g).to(DEV)
    txt = torch.randn(1, 16, cfg.context_dim, generator=g).to(DEV, torch.bfloat16)
    t = torch.full((1,), 0.5, device=DEV)
    results = []
    for sharded in (False, True):
        m = QwenImageDiT(cfg, torch.bfloat16, DEV).init_weights(0)
        ctx = None
        if sharded:
            ctx = FSDPContext(mode="nccl", device=torch.device(DEV, 0))
            n = shard_model(m, ctx, min_params=1 << 12)
            assert n > 20 and any(isinstance(x, ShardedLinear) for x in m.modules())
        params = [p for p in m.parameters() if p.numel() > 0]
        for p in params:
            p.requires_grad_(True)
        opt = FusedAdamW(params, lr=1e-3, weight_decay=0.01, max_grad_norm=0.0, master_weights=True)
        m.gradient_checkpointing = True
        m.train()
        losses = []
        for _ in range(3):
            opt.zero_grad(set_to_none=True)
            xt, target = O.flow_match(x0, eps, t)
            loss = O.mse_loss(m(xt.to(torch.bfloat16), txt, t, (8, 8)), target)
            loss.backward()
            opt.step()
            if ctx is not None:
                ctx.step(lr=1e-3)
            losses.append(float(loss))
        blk = m.transformer_blocks[1].attn.to_q
        w = blk.inner.full_master() if sharded else blk.weight.detach().float()
        results.append((losses, w))
    native.check_status()
    (l0, w0), (l1, w1) = results
    assert all(abs(a - b) <= 0.02 * abs(a) + 1e-3 for a, b in zip(l0, l1)), (l0, l1)
    assert l0[-1] < l0[0]
    assert _cos(w1, w0) > 0.9999 and float((w1 - w0.to(w1.device)).abs().max()) < 2e-2


def test_cuda_graph_replay_equals_eager_forward_bitwise():
    """Capture gate for inference: a replayed graph of the tiny MMDiT forward reproduces the eager result bit for bit."""
    from mojodiffusion_b200.models.mmdit import MMDiT, tiny_mmdit_config
    from mojodiffusion_b200.utils.cuda_graph import graphs_equal_eager
    cfg = tiny_mmdit_config()
    m = MMDiT(cfg, torch.bfloat16, DEV).init_weights(0).eval()
    g = torch.Generator().manual_seed(11)
    img = torch.randn(1, 64, cfg.in_channels, generator=g).to(DEV, torch.bfloat16)
    txt = torch.randn(1, 16, cfg.context_dim, generator=g).to(DEV, torch.bfloat16)
    y = torch.randn(1, cfg.vec_dim, generator=g).to(DEV, torch.bfloat16)
    t = torch.full((1,), 0.4, device=DEV)
    ids = MMDiT.make_ids(8, 8, 16, DEV)
    same, err = graphs_equal_eager(lambda a, b, c, d: m(a, b, c, d, None, ids=ids), [img, txt, t, y])
    native.check_status()
    assert same, err


def test_cuda_graph_train_step_matches_eager():
    """Forward + backward captured as one graph (checkpointed blocks recompute inside the captured backward), optimizer
    after the replay: three LoRA steps give the losses and adapter weights of the eager trainer."""
    from mojodiffusion_b200.models.mmdit import MMDiT, tiny_mmdit_config
    from mojodiffusion_b200.training import lora as L
    from mojodiffusion_b200.training.optim import FusedAdamW
    from mojodiffusion_b200.training.trainer import FlowMatchTrainer
    cfg = tiny_mmdit_config()
    g = torch.Generator().manual_seed(12)
    x0 = torch.randn(1, 64, cfg.in_channels, generator=g).to(DEV)
    txt = torch.randn(1, 16, cfg.context_dim, generator=g).to(DEV, torch.bfloat16)
    y = torch.randn(1, cfg.vec_dim, generator=g).to(DEV, torch.bfloat16)
    out = []
    for graphed in (False, True):
        m = MMDiT(cfg, torch.bfloat16, DEV).init_weights(0)
        slots = L.inject_flux_lora(m, rank=8, alpha=8.0)
        params = L.lora_parameters(slots)
        m.gradient_checkpointing = True
        m.train()
        tr = FlowMatchTrainer(m, params, FusedAdamW(params, lr=1e-3, max_grad_norm=1.0), use_cuda_graph=graphed)
        losses = [float(tr.step(x0, txt, y, hw=(8, 8))) for _ in range(4)]
        out.append((losses, torch.cat([p.detach().float().flatten() for p in params])))
        if graphed:
            assert tr._graphed is not None and tr._graphed.graph is not None
    native.check_status()
    (l0, w0), (l1, w1) = out
    assert all(abs(a - b) <= 2e-3 * abs(a) + 1e-4 for a, b in zip(l0, l1)), (l0, l1)
    assert _cos(w1, w0) > 0.9999


def test_more_video_and_image_families_on_native_kernels():
    """Ideogram-4, HunyuanVideo-1.5, Kandinsky-5, Cosmos-Predict2.5 and Wan-VACE (tiny configurations) in bf16 on the
    sm_100a kernels against their fp32 CPU forward."""
    from mojodiffusion_b200.models.cosmos import CosmosDiT, tiny_cosmos_config
    from mojodiffusion_b200.models.hunyuan15 import Hunyuan15DiT, tiny_hunyuan15_config
    from mojodiffusion_b200.models.ideogram4 import Ideogram4DiT, tiny_ideogram4_config
    from mojodiffusion_b200.models.kandinsky5 import Kandinsky5DiT, tiny_kandinsky5_config
    from mojodiffusion_b200.models.wan import WanVaceDiT, tiny_wan_vace_config
    g = torch.Generator().manual_seed(11)
    rn = lambda *s: torch.randn(*s, generator=g)
    ci = tiny_ideogram4_config()
    L = 48
    ind = torch.tensor([[3] * 16 + [2] * 24 + [0] * 8])
    pos = torch.stack([torch.zeros(L), torch.arange(L).float() * 5, torch.arange(L).float()], 1)
    _gpu_vs_cpu(lambda dt, dev: Ideogram4DiT(ci, dt, dev), (rn(1, L, ci.in_channels), rn(1, L, ci.llm_dim), torch.tensor([0.4]), ind, pos), cos_min=0.99)
    ch = tiny_hunyuan15_config()
    _gpu_vs_cpu(lambda dt, dev: Hunyuan15DiT(ch, dt, dev), (rn(1, ch.in_channels, 2, 4, 8), rn(1, 16, ch.hidden), torch.tensor([0.3])), cos_min=0.99)
    ck = tiny_kandinsky5_config()
    _gpu_vs_cpu(lambda dt, dev: Kandinsky5DiT(ck, dt, dev), (rn(1, ck.in_visual_dim, 2, 8, 8), rn(1, 16, ck.in_text_dim), rn(1, ck.in_text_dim2),
                                                           torch.tensor([417.0])), cos_min=0.99)
    cc = tiny_cosmos_config()
    _gpu_vs_cpu(lambda dt, dev: CosmosDiT(cc, dt, dev), (rn(1, cc.in_channels, 2, 8, 8), rn(1, 16, cc.text_in_dim), torch.tensor([0.6])), cos_min=0.99)
    cv = tiny_wan_vace_config()
    m32 = WanVaceDiT(cv, torch.float32, "cpu").init_weights(0)
    with torch.no_grad():                              # give the zero-initialised control projections weight so the branch acts
        for blk in m32.vace_blocks:
            for lin in (blk.before_proj, blk.after_proj):
                if lin is not None:
                    lin.weight.copy_(torch.randn(lin.weight.shape, generator=g) * 0.05)
    mg = WanVaceDiT(cv, torch.bfloat16, DEV)
    mg.load_state_dict({k: v.to(torch.bfloat16) for k, v in m32.state_dict().items()})
    m32.load_state_dict({k: v.float() for k, v in mg.state_dict().items()})
    z, txt, t, ctl = rn(1, cv.in_dim, 2, 8, 8), rn(1, 16, cv.text_dim), torch.tensor([0.5]), rn(1, cv.vace_in_dim, 2, 8, 8)
    with torch.no_grad():
        want, base = m32(z, txt, t, control=ctl), m32(z, txt, t)
        got = mg(z.to(DEV), txt.to(DEV), t.to(DEV), control=ctl.to(DEV))
    native.check_status()
    assert (want - base).abs().max() > 1e-3 and _cos(got, want) >= 0.99


def test_moe_audio_spine_and_krea2_families_on_native_kernels():
    """Nucleus-Image (expert-choice MoE), ACE-Step (audio), HiDream-O1 (language-model spine), Krea-2, Lens, Z-Image L2P, Boogu-Image, MagiHuman, Lance T2V and SenseNova-U1 (tiny configurations,
    head width 64) in bf16 on the sm_100a kernels against their fp32 CPU forward."""
    import dataclasses
    from mojodiffusion_b200.models.acestep import AceStepDiT, tiny_acestep_config
    from mojodiffusion_b200.models.hidream_o1 import HiDreamO1, build_mrope_positions, tiny_hidream_o1_config
    from mojodiffusion_b200.models.krea2 import Krea2DiT, krea2_positions, tiny_krea2_config
    from mojodiffusion_b200.models.nucleus import NucleusDiT, tiny_nucleus_config
    g = torch.Generator().manual_seed(12)
    rn = lambda *s: torch.randn(*s, generator=g)
    cn = tiny_nucleus_config()
    _gpu_vs_cpu(lambda dt, dev: NucleusDiT(cn, dt, dev), (rn(1, 8 * 8, cn.in_channels), rn(1, 16, cn.joint_dim), torch.tensor([0.3])),
                cos_min=0.99, grid=(1, 8, 8))
    ca = dataclasses.replace(tiny_acestep_config(), hidden=256, head_dim=64)
    _gpu_vs_cpu(lambda dt, dev: AceStepDiT(ca, dt, dev), (rn(1, 32, ca.acoustic_dim), rn(1, 32, ca.in_channels - ca.acoustic_dim), rn(1, 8, ca.hidden),
                                                         torch.tensor([0.7]), torch.tensor([0.2])), cos_min=0.99)
    ck = dataclasses.replace(tiny_krea2_config(), features=256, txtdim=128)
    gh, gw, Lt = 8, 8, 16
    pos = krea2_positions(Lt, gh, gw)
    _gpu_vs_cpu(lambda dt, dev: Krea2DiT(ck, dt, dev), (rn(1, gh * gw, ck.patch_dim), rn(1, Lt, ck.txtlayers, ck.txtdim), torch.tensor([0.6]), pos),
                cos_min=0.99)
    from mojodiffusion_b200.models.lens import LensDiT, tiny_lens_config
    from mojodiffusion_b200.models.zimage_l2p import ZImageL2P, tiny_zimage_l2p_config
    cl = tiny_lens_config()
    _gpu_vs_cpu(lambda dt, dev: LensDiT(cl, dt, dev), (rn(1, 8 * 8, cl.in_channels), rn(1, 16, 4, cl.text_hidden), torch.tensor([0.4])), cos_min=0.99, hw=(8, 8))
    cz = tiny_zimage_l2p_config()
    _gpu_vs_cpu(lambda dt, dev: ZImageL2P(cz, dt, dev, (64, 64, 128, 128)), (rn(1, 3, 64, 64), rn(1, 16, cz.cap_dim), torch.tensor([0.6])), cos_min=0.99)
    from mojodiffusion_b200.models.boogu import BooguDiT, tiny_boogu_config
    cb = tiny_boogu_config()
    _gpu_vs_cpu(lambda dt, dev: BooguDiT(cb, dt, dev), (rn(1, cb.in_channels, 16, 16), rn(1, 16, cb.instruction_dim), torch.tensor([0.3])), cos_min=0.99)
    from mojodiffusion_b200.models.magihuman import MagiHumanDiT, tiny_magihuman_config
    cm = dataclasses.replace(tiny_magihuman_config(), hidden_size=256, head_dim=64, rope_dim=48, rope_bands=8)
    V, A, T = 32, 8, 8
    coords = torch.cat((torch.stack(torch.meshgrid(torch.arange(2.0), torch.arange(4.0), torch.arange(4.0), indexing="ij"), -1).reshape(V, 3),
                        torch.stack((torch.arange(A).float(), torch.zeros(A), torch.zeros(A)), 1),
                        torch.stack((torch.arange(T).float(), torch.zeros(T), torch.zeros(T)), 1)), 0)
    coords = torch.cat((coords, torch.tensor([[2.0, 4.0, 4.0, 2.0, 8.0, 8.0]]).expand(V + A + T, 6)), 1)
    _gpu_vs_cpu(lambda dt, dev: MagiHumanDiT(cm, dt, dev), (rn(V, cm.video_in), rn(A, cm.audio_in), rn(T, cm.text_in), coords), cos_min=0.99)
    from mojodiffusion_b200.models.lance import LanceT2V, build_lance_input, tiny_lance_config
    from mojodiffusion_b200.models.sensenova_u1 import SenseNovaU1, tiny_sensenova_u1_config
    for make, run in ((lambda dt, dev: LanceT2V(tiny_lance_config(), dt, dev),
                       lambda mod, dev: mod(build_lance_input(tiny_lance_config(), [3, 4, 5, 6], 2, 2, 3), xl.to(dev), torch.tensor([0.4], device=dev))),
                      (lambda dt, dev: SenseNovaU1(dataclasses.replace(tiny_sensenova_u1_config(), head_dim=64), dt, dev),
                       lambda mod, dev: mod.predict_clean(xs.to(dev), 0.3, mod.forward_und([5, 9, 2, 7]), 4))):
        xl, xs = rn(12, tiny_lance_config().patch_latent_dim), rn(1, 3, 32, 32)
        m32 = make(torch.float32, "cpu").init_weights(0)
        mg = make(torch.bfloat16, DEV)
        mg.load_state_dict({k: v.to(torch.bfloat16) for k, v in m32.state_dict().items()})
        m32.load_state_dict({k: v.float() for k, v in mg.state_dict().items()})
        with torch.no_grad():
            want, got = run(m32, "cpu"), run(mg, DEV)
        native.check_status()
        assert torch.isfinite(got.float()).all() and _cos(got, want) >= 0.99
    chd = tiny_hidream_o1_config()
    chd = dataclasses.replace(chd, spine=dataclasses.replace(chd.spine, hidden_size=256, head_dim=64))
    ids = [1, 2, chd.tms_token_id, 3, chd.vision_start_token_id]
    L = 16
    ppos = build_mrope_positions(ids + [chd.image_token_id] * L, chd.image_token_id, 4, 4, 10)
    m32 = HiDreamO1(chd, torch.float32, "cpu").init_weights(0)
    mg = HiDreamO1(chd, torch.bfloat16, DEV)
    mg.load_state_dict({k: v.to(torch.bfloat16) for k, v in m32.state_dict().items()})
    m32.load_state_dict({k: v.float() for k, v in mg.state_dict().items()})
    patches = rn(1, L, chd.patch_dim)
    want = m32(ids, patches, ppos, len(ids), 0.4)
    got = mg(ids, patches.to(DEV), ppos, len(ids), 0.4)
    native.check_status()
    assert _cos(got[:, len(ids):], want[:, len(ids):]) >= 0.99
