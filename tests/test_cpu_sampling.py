"""Schedulers and solvers against closed forms: exact ODE solutions, coefficient identities, admission rules."""
import json
import math

import torch

from mojodiffusion_b200.sampling import ddpm, guidance, inpaint, ltx2, multistep, registry
from mojodiffusion_b200.sampling import flow_match as fm


def test_sdxl_euler_schedule_constants():
    s = ddpm.SDXLEulerScheduler(30)
    assert len(s.timesteps) == 30 and s.timesteps[0] == 29 * 33 + 1 and s.timesteps[-1] == 1
    ac = ddpm.alphas_cumprod()
    assert abs(s.sigmas[0] - math.sqrt((1 - float(ac[s.timesteps[0]])) / float(ac[s.timesteps[0]]))) < 1e-12
    assert s.sigmas[-1] == 0.0 and all(a > b for a, b in zip(s.sigmas, s.sigmas[1:]))
    assert abs(s.init_noise_sigma - math.sqrt(s.sigmas[0] ** 2 + 1)) < 1e-12
    b = ddpm.scaled_linear_betas()
    assert abs(float(b[0]) - 0.00085) < 1e-9 and abs(float(b[-1]) - 0.012) < 1e-9
    # an exact-eps oracle: x_sigma = x0 + sigma eps  -> Euler recovers x0
    x0, eps = torch.randn(1, 4, 8, 8), torch.randn(1, 4, 8, 8)
    out = ddpm.euler_eps_sample(lambda xin, t: eps, eps, s)
    # start = eps * sqrt(sig0^2+1); trajectory subtracts sig0*eps in total
    assert torch.allclose(out, eps * (s.init_noise_sigma - s.sigmas[0]), atol=1e-4)
    noisy, tgt = ddpm.ddpm_add_noise(x0, eps, torch.tensor([500]))
    a = float(ac[500])
    assert torch.allclose(noisy, math.sqrt(a) * x0 + math.sqrt(1 - a) * eps, atol=1e-5) and torch.equal(tgt, eps)


def _flow_x0_oracle(x0_true):
    # perfect data predictor for x_t = (1-s) x0 + s eps
    return lambda x, i: x0_true


def test_dpmpp_2m_and_unipc_solve_flow_ode_exactly_for_constant_x0():
    sig = fm.shifted_sigmas(8, 3.0)
    al = [1 - s for s in sig]
    x0 = torch.randn(2, 16)
    eps = torch.randn(2, 16)
    start = (1 - sig[0]) * x0 + sig[0] * eps
    for solver in (multistep.DPMPP2M(al, sig), multistep.UniPCMultistep(al, sig, order=2)):
        out = multistep.sample_multistep(_flow_x0_oracle(x0), start.clone(), solver, 8)
        assert torch.allclose(out, x0, atol=1e-4)
    # one interior step of DPM++ 2M with constant x0 lands exactly on the x_t line
    sol = multistep.DPMPP2M(al, sig)
    x1 = sol.step(start, x0, 0)
    assert torch.allclose(x1, (1 - sig[1]) * x0 + sig[1] * eps, atol=1e-5)


def test_res2s_coefficients_and_samplers():
    assert abs(ltx2.phi(1, 1e-9) - 1.0) < 1e-6 and abs(ltx2.phi(2, 1e-9) - 0.5) < 1e-6
    assert abs(ltx2.phi(1, -0.7) - (math.exp(-0.7) - 1) / -0.7) < 1e-12
    h, a21, b1, b2, sub = ltx2.res2s_coefficients(0.8, 0.4)
    assert abs(h - math.log(2)) < 1e-12 and abs(sub - math.sqrt(0.32)) < 1e-12
    assert abs((b1 + b2) - ltx2.phi(1, -h)) < 1e-12                 # consistency: weights sum to phi_1
    x0 = torch.randn(1, 10, 8)
    eps = torch.randn(1, 10, 8)
    v = eps - x0                                                  # exact velocity of the straight path
    sig = fm.ltx2_linear_quadratic_sigmas(12)
    out = ltx2.euler_ltx2_sample(lambda x, s: v, eps.clone(), sig)
    assert torch.allclose(out, x0, atol=1e-4)
    out = ltx2.res2s_sample(lambda x, s: (x - x0) / max(s, 1e-9), eps.clone(), sig)     # v from a perfect denoiser
    assert torch.allclose(out, x0, atol=1e-3)
    ar, sd, su = ltx2.sde_coefficients(0.5, 0.5)
    assert abs(su - 0.25) < 1e-12 and abs(ar - (0.5 + math.sqrt(0.25 - 0.0625))) < 1e-12
    assert ltx2.DISTILLED_STAGE1[0] == 1.0 and ltx2.DISTILLED_STAGE1[-1] == 0.0


def test_guidance_identities():
    vc, vu = torch.randn(2, 7, 5), torch.randn(2, 7, 5)
    assert torch.allclose(guidance.cfg_textbook(vc, vu, 1.0), vc, atol=1e-6)
    assert torch.allclose(guidance.cfg_cond_anchored(vc, vu, 0.0), vc)
    r = guidance.cfg_true_with_norm_rescale(vc, vu, 4.0)
    assert torch.allclose(r.norm(dim=-1), vc.norm(dim=-1), rtol=1e-4)
    assert torch.allclose(guidance.cfg_star_rescale(vc, vc, 3.0), vc, atol=1e-5)
    assert torch.allclose(guidance.stg_combine(vc, vu, vc, 1.0, 2.0), vc, atol=1e-6)
    assert guidance.stg_skip_mask(6, [2, 4]).tolist() == [1, 1, 0, 1, 0, 1]
    z = guidance.nag_attention_guidance(vc, vc, 5.0)
    assert torch.allclose(z, vc, atol=1e-5)


def test_inpaint_and_variation_helpers():
    lat, noise = torch.randn(1, 4, 8, 8), torch.randn(1, 4, 8, 8)
    sig = fm.shifted_sigmas(10, 1.0)
    x, first = inpaint.img2img_start(lat, noise, sig, 0.6)
    assert first == 4 and torch.allclose(x, (1 - sig[4]) * lat + sig[4] * noise)
    mask = torch.zeros(1, 1, 8, 8)
    mask[..., :4] = 1
    b = inpaint.inpaint_blend(torch.ones_like(lat), lat, noise, mask, 0.0)
    assert torch.allclose(b[..., 4:], lat[..., 4:]) and torch.allclose(b[..., :4], torch.ones_like(lat)[..., :4])
    a = inpaint.variation_noise((4, 16), 1, 2, 0.0)
    c = inpaint.variation_noise((4, 16), 1, 2, 1.0)
    assert torch.equal(a, torch.randn((4, 16), generator=torch.Generator().manual_seed(1)))
    assert torch.allclose(c, torch.randn((4, 16), generator=torch.Generator().manual_seed(2)), atol=1e-5)
    m = inpaint.variation_noise((4, 16), 1, 2, 0.3)
    assert abs(float(m.norm()) - float(a.norm())) < 0.15 * float(a.norm())
    assert inpaint.quantize_resolution(1000, 1032, 16) == (992, 1024) and inpaint.quantize_resolution(1016, 1030, 16) == (1024, 1024)  # ties to even
    toks, ids = inpaint.pack_reference_tokens(torch.zeros(1, 4, 8), torch.zeros(4, 3), torch.ones(1, 6, 8), (2, 3))
    assert toks.shape == (1, 10, 8) and ids[4:, 0].tolist() == [1.0] * 6 and ids[-1].tolist() == [1.0, 1.0, 2.0]


def test_registry_admission():
    assert registry.normalize_sampler("DPM++ 2M") == "dpmpp_2m" and registry.normalize_sampler("UniPC") == "uni_pc"
    ok, why = registry.admit("flux", "euler", "simple")
    assert ok
    ok, why = registry.admit("flux", "dpmpp_2m", "simple")
    assert not ok and "not implemented" in why
    assert not registry.admit("flux", "made_up", "simple")[0] and not registry.admit("nope", "euler", "simple")[0]
    j = json.loads(registry.registry_json())
    assert j["schema"] == "serenity.samplers.v1" and "res_2s" in j["samplers"]
    k = registry.karras_sigmas(5, 0.03, 14.6)
    assert abs(k[0] - 14.6) < 1e-9 and abs(k[-2] - 0.03) < 1e-9 and k[-1] == 0.0


def test_family_schedules():
    """Ideogram-4, Cosmos, ACE-Step, Lens, Krea-2 and HiDream-O1 schedule tables against their closed forms and anchors."""
    import math
    import torch
    from mojodiffusion_b200.sampling import family_schedules as S
    # Ideogram-4: the median of the logit-normal sits at 1 - sigmoid(mean); the ends are clamped by the log-SNR window
    mean = S.ideogram4_schedule_mean(1024, 1024)
    assert abs(mean - (1.0 + 0.5 * math.log(4.0))) < 1e-12
    assert abs(S.ideogram4_logitnormal(0.5, mean) - (1 - 1 / (1 + math.exp(-mean)))) < 1e-12
    lv = S.ideogram4_levels(10, 1024, 1024)
    assert len(lv) == 11 and all(a > b for a, b in zip(lv, lv[1:]))
    assert abs(lv[0] - 1 / (1 + math.exp(-7.5))) < 1e-12 and abs(lv[-1] - 1 / (1 + math.exp(9.0))) < 1e-12
    assert abs(S.ideogram4_logitnormal(0.975, 0.0) - (1 - 1 / (1 + math.exp(-1.959963984540054)))) < 1e-9
    # Cosmos: first sigma 0.9998 at shift 5, 35 steps
    cs = S.cosmos_rf_sigmas(35, 5.0)
    assert len(cs) == 36 and cs[-1] == 0.0 and abs(cs[0] - 5 * 0.999 / (1 + 4 * 0.999)) < 1e-12 and abs(cs[0] - 0.9998) < 1e-4
    assert S.cosmos_timesteps(cs)[0] == cs[0] * 1000 and len(S.cosmos_timesteps(cs)) == 35
    # ACE-Step
    a = S.acestep_sigmas(8, 3.0)
    assert len(a) == 9 and a[0] == 1.0 and a[-1] == 0.0 and abs(a[4] - 3 * 0.5 / (1 + 2 * 0.5)) < 1e-12
    x, v = torch.ones(3), torch.full((3,), 2.0)
    assert torch.allclose(S.acestep_euler_step(x, v, 0.8, 0.5), x - v * 0.3)
    # Lens: documented anchor mu(4096 tokens, 20 steps) = 2.1980220725551165
    assert abs(S.lens_empirical_mu(S.lens_image_seq_len(1024, 1024), 20) - 2.1980220725551165) < 1e-12
    ls = S.lens_sigmas(20, 4096)
    assert len(ls) == 20 and ls[0] == 1.0 and all(p > q for p, q in zip(ls, ls[1:]))
    e = math.exp(2.1980220725551165)
    assert abs(ls[-1] - e * 0.05 / (e * 0.05 + 0.95)) < 1e-12
    assert abs(S.lens_empirical_mu(5000, 7) - (0.00016927 * 5000 + 0.45666666)) < 1e-12
    # Krea-2: the line through (256 tokens, 0.5) and (6400 tokens, 1.15)
    assert abs(S.krea2_mu(256) - 0.5) < 1e-12 and abs(S.krea2_mu(6400) - 1.15) < 1e-12
    kt = S.krea2_timesteps(S.krea2_packed_seq_len(1024, 1024), 4)
    mu = S.krea2_mu(4096)
    assert kt[0] == 1.0 and kt[-1] == 0.0 and abs(kt[2] - math.exp(mu) / (math.exp(mu) + 1.0)) < 1e-12
    assert abs(S.krea2_timesteps(4096, 4, mu=1.15)[2] - math.exp(1.15) / (math.exp(1.15) + 1)) < 1e-12
    assert torch.allclose(S.krea2_cfg(torch.tensor([2.0]), torch.tensor([1.0]), 3.0), torch.tensor([5.0]))
    # HiDream-O1
    d = S.HiDreamO1Scheduler.dev()
    assert len(d.timesteps) == 28 and d.sigmas[0] == 0.999 and d.sigmas[-1] == 0.0 and d.flash
    f = S.HiDreamO1Scheduler.full(5, 3.0)
    assert abs(f.sigmas[0] - 1.0) < 1e-12 and abs(f.sigmas[4] - 3 * 0.001 / (1 + 2 * 0.001)) < 1e-12 and not f.flash
    smp, mo, nz = torch.randn(4, 8), torch.randn(4, 8), torch.randn(4, 8) * 3
    assert torch.allclose(f.step(mo, 1, smp), smp + (f.sigmas[2] - f.sigmas[1]) * mo)
    out = d.step(mo, 0, smp, nz, s_noise=1.0, noise_clip_std=1.0)
    clip = float(nz.std(unbiased=False))
    assert torch.allclose(out, d.sigmas[1] * nz.clamp(-clip, clip) + (1 - d.sigmas[1]) * (smp - d.sigmas[0] * mo), atol=1e-6)


def test_pid_lance_samplers_and_lance_kv_plan():
    import dataclasses
    import pytest
    import torch
    from mojodiffusion_b200.runtime import lance_kv_plan as K
    from mojodiffusion_b200.sampling import family_schedules as S
    # PiD: with the exact velocity of a straight path and zero fresh noise the sample lands on the data
    x0, eps = torch.rand(1, 3, 4, 4) * 1.6 - 0.8, torch.randn(1, 3, 4, 4)
    seen = []

    def model(x, t):
        seen.append(t)
        return (x - x0) / (t / 1000.0)                 # v with x = x0 + t (eps' ) for whichever noise is in x
    out = S.pid_distill_sample(model, 0.001 * x0 + 0.999 * eps, lambda: torch.zeros_like(x0))
    assert seen == [999.0, 866.0, 634.0, 342.0] and torch.allclose(out, x0, atol=1e-5)
    assert S.pid_distill_sample(lambda x, t: torch.zeros_like(x), torch.full((2,), 5.0), lambda: torch.zeros(2), times=(0.5, 0.0)).max() == 1.0
    # Lance: schedule, renormalised guidance, Euler step
    lt = S.lance_times(4, 3.0)
    assert lt[0] == 1.0 and lt[-1] == 0.0 and abs(lt[2] - 3 * 0.5 / 2.0) < 1e-12
    vc, vu = torch.tensor([3.0, 4.0]), torch.tensor([0.0, 0.0])
    g = S.lance_cfg_renorm(vc, vu, 5.0)                # guided norm 25 -> ratio 0.2 -> back to norm 5
    assert torch.allclose(g, vc, atol=1e-5)
    assert torch.allclose(S.lance_cfg_renorm(vc, vu, 0.5, 0.0, 1.0), vc * 0.5)        # ratio 2 clamped to 1
    assert torch.allclose(S.lance_denoise_step(torch.ones(2), torch.ones(2), 0.8, 0.5), torch.full((2,), 0.7))
    # KV plan: 5 text tokens, 2 x 2 x 3 latent grid
    gen = 12
    total = 5 + 1 + gen + 1
    inp = K.LanceInput(list(range(total)), [0] * total, [0] * total, [0] * total, 5, 6, gen, list(range(gen)))
    plan = K.text_drop_plan(inp)
    K.validate_plan(inp, plan, 4, (2, 2, 3))
    c, u = K.layer_call(plan, K.BRANCH_COND, 3), K.layer_call(plan, K.BRANCH_TEXT_UNCOND, 3)
    assert (c.source_query_start, c.packed_query_start, c.attention_kv_len, c.prefix_cache_write_len) == (5, 5, total, 5)
    assert (u.source_query_start, u.packed_query_start, u.attention_kv_len, u.prefix_cache_write_len) == (5, 0, gen + 2, 0)
    assert plan.total_kv_bytes(4, 8, 128) == 5 * 8 * 128 * 2 * 2 * 4
    with pytest.raises(ValueError):
        K.validate_plan(inp, plan, 4, (2, 2, 2))
    with pytest.raises(ValueError):
        K.validate_input(dataclasses.replace(inp, gen_start=5))
    with pytest.raises(ValueError):
        K.layer_call(plan, 2, 0)
