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
