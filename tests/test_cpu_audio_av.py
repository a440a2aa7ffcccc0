"""CPU tests of the LTX-2 audio / video stack: joint AV transformer, audio VAE, BigVGAN-v2 vocoder with bandwidth
extension, anti-aliased activation and band-limited resampling."""
import math

import pytest
import torch

from mojodiffusion_b200.models import audio_vae as AV
from mojodiffusion_b200.models import ltx2_av as L
from mojodiffusion_b200.models import vocoder as V
from mojodiffusion_b200.ops import audio as A


def _av_inputs(cfg, B=2, grid=(2, 3, 4), Na=10, T=12):
    g = torch.Generator().manual_seed(1)
    Nv = grid[0] * grid[1] * grid[2]
    vx = torch.randn(B, Nv, cfg.in_channels, generator=g)
    ax = torch.randn(B, Na, cfg.audio_in_channels, generator=g)
    text = torch.randn(B, T, cfg.context_dim, generator=g)
    t = torch.tensor([0.3, 0.7])[:B]
    return vx, ax, text, t, grid


def test_ltx2_av_forward_shapes_cross_modal_and_nag():
    cfg = L.tiny_ltx2_av_config()
    m = L.LTX2AVDiT(cfg, dtype=torch.float32)
    with torch.no_grad():
        m.init_weights(0)
        vx, ax, text, t, grid = _av_inputs(cfg)
        v, a = m(vx, ax, text, t, grid)
        assert v.shape == vx.shape and a.shape == ax.shape
        assert torch.isfinite(v).all() and torch.isfinite(a).all()
        v2, a2 = m(vx, ax, text, t, grid, skip_cross_modal=True)
        assert (v - v2).abs().max() > 1e-5 and (a - a2).abs().max() > 1e-5      # the cross-modal sub-layers contribute
        neg = torch.randn(text.shape, generator=torch.Generator().manual_seed(5))
        v3, a3 = m(vx, ax, text, t, grid, nag=(neg, 4.0, 2.5, 0.25))
        assert torch.isfinite(v3).all() and (v - v3).abs().max() > 1e-6
        # audio changes reach the video output only through the cross-modal attention
        ax2 = ax + 1.0
        v4, _ = m(vx, ax2, text, t, grid)
        v5, _ = m(vx, ax2, text, t, grid, skip_cross_modal=True)
        assert (v4 - v).abs().max() > 1e-6
        assert torch.equal(v5, v2)


def test_ltx2_av_gradients_and_adapter_prefixes_resolve():
    cfg = L.tiny_ltx2_av_config()
    m = L.LTX2AVDiT(cfg, dtype=torch.float32)
    with torch.no_grad():
        m.init_weights(0)
    vx, ax, text, t, grid = _av_inputs(cfg, B=1)
    v, a = m(vx, ax, text, t[:1], grid)
    (v.square().mean() + a.square().mean()).backward()
    got = [n for n, p in m.named_parameters() if p.grad is not None and p.grad.abs().sum() > 0]
    assert any("audio_to_video_attn" in n for n in got) and any("video_to_audio_attn" in n for n in got)
    mods = dict(m.named_modules())
    prefixes = L.ltx2_av_lora_prefixes(cfg.depth)
    assert len(prefixes) == cfg.depth * (6 * 4 + 4 + 4)
    for p in prefixes:
        assert p.removeprefix("diffusion_model.") in mods, p


def test_activation1d_keeps_length_and_matches_snake_on_band_limited_input():
    t = torch.arange(400) / 400.0
    x = (0.5 * torch.sin(2 * math.pi * 3 * t))[None, None].repeat(1, 2, 1)
    al, be = torch.tensor([0.1, -0.2]), torch.tensor([0.0, 0.3])
    y = A.activation1d(x, al, be)
    assert y.shape == x.shape
    ref = A.snake(x, al, be)
    assert (y - ref)[..., 20:-20].abs().max() < 2e-3           # slow signal: filtering is transparent away from the edges
    f = A.kaiser_sinc_filter1d(0.25, 0.3, 12)
    assert abs(float(f.sum()) - 1.0) < 1e-6 and torch.allclose(f, f.flip(0), atol=1e-7)


def test_resample_hann_matches_torchaudio_rule():
    t = torch.arange(1600) / 16000.0
    s = torch.sin(2 * math.pi * 440 * t)[None, None]
    u = A.resample_hann(s, 16000, 48000)
    assert u.shape[-1] == 4800
    t3 = torch.arange(4800) / 48000.0
    assert (u[0, 0, 100:-100] - torch.sin(2 * math.pi * 440 * t3)[100:-100]).abs().max() < 1e-3
    d = A.resample_hann(u, 48000, 16000)
    assert d.shape[-1] == 1600 and (d - s)[..., 50:-50].abs().max() < 2e-3
    ta = pytest.importorskip("torchaudio")
    assert (ta.functional.resample(s, 16000, 48000) - u).abs().max() < 1e-5


def test_audio_vae_shapes_causality_and_statistics():
    cfg = AV.tiny_audio_vae_config()
    vae = AV.AudioVAE(cfg)
    with torch.no_grad():
        vae.init_weights(0)
        z = torch.randn(1, cfg.latent_channels, 5, cfg.mel_bins_latent)
        mel = vae.decode(z)
        assert mel.shape == (1, 2, 2 * 5 - 1, 2 * cfg.mel_bins_latent)
        z2 = z.clone()
        z2[:, :, 3:] += 1.0                                    # a later latent frame cannot change earlier mel frames
        mel2 = vae.decode(z2)
        assert torch.allclose(mel[:, :, :4], mel2[:, :, :4], atol=1e-6) and not torch.allclose(mel, mel2)
        n = cfg.latent_channels * cfg.mel_bins_latent
        getattr(vae.per_channel_statistics, "mean-of-means").copy_(torch.linspace(-1, 1, n))
        getattr(vae.per_channel_statistics, "std-of-means").copy_(torch.linspace(0.5, 2, n))
        assert torch.allclose(vae.normalize(vae.un_normalize(z)), z, atol=1e-5)
        u = vae.un_normalize(torch.zeros_like(z))              # statistic index = channel * bins + bin
        assert abs(float(u[0, 1, 0, 2]) - float(torch.linspace(-1, 1, n)[1 * cfg.mel_bins_latent + 2])) < 1e-6
        lat = vae.encode(torch.randn(1, 2, 9, 2 * cfg.mel_bins_latent))
        assert lat.shape == (1, cfg.latent_channels, 5, cfg.mel_bins_latent)
    full = AV.ltx2_audio_vae_config()
    assert (full.latent_channels, full.mel_bins_latent, full.base_channels, full.ch_mult) == (8, 16, 128, (1, 2, 4))


def test_full_size_audio_decoder_time_and_frequency_growth():
    vae = AV.AudioVAE(AV.ltx2_audio_vae_config(), with_encoder=False)
    with torch.no_grad():
        out = vae.decode(torch.randn(1, 8, 4, 16))
    assert out.shape == (1, 2, 4 * 4 - 3, 64)
    keys = set(vae.state_dict())
    assert "decoder.up.2.upsample.conv.conv.weight" in keys and "decoder.up.0.block.2.conv2.conv.weight" in keys
    assert "decoder.up.1.block.0.nin_shortcut.conv.weight" in keys and "per_channel_statistics.mean-of-means" in keys


def test_bigvgan2_and_bandwidth_extension():
    voc = V.tiny_bigvgan2_config(8, (2, 2))
    bwe = V.tiny_bigvgan2_config(2 * 8, (4, 3))           # mel hop 4 x rate ratio 3
    m = V.VocoderWithBWE(voc, bwe, 16000, 48000, n_fft=32, hop=4, n_mels=8)
    keys = set(m.state_dict())
    for k in ("vocoder.conv_pre.weight", "vocoder.ups.0.weight", "vocoder.resblocks.0.acts1.0.act.alpha",
              "vocoder.resblocks.0.acts2.1.downsample.lowpass.filter", "vocoder.act_post.upsample.filter",
              "bwe_generator.conv_post.weight", "mel_stft.mel_basis", "mel_stft.stft_fn.forward_basis"):
        assert k in keys, k
    mel = torch.randn(1, 2, 10, 4)
    low = m.vocoder(mel)
    assert low.shape == (1, 2, 10 * 4)
    out = m(mel)
    assert out.shape == (1, 2, 40 * 3) and out.abs().max() <= 1.0
    full, fb = V.ltx2_vocoder_config(), V.ltx2_bwe_config()
    assert math.prod(full.upsample_rates) == 160 and math.prod(fb.upsample_rates) == 240   # mel hop 160 @16 kHz; 80 * 3 @48 kHz


def test_mel_stft_by_convolution_matches_fft():
    ms = V.MelSTFT(n_fft=64, hop=16, n_mels=8, sample_rate=16000)
    x = torch.randn(1, 1, 640, generator=torch.Generator().manual_seed(3))
    got = ms(x)[0, 0]
    xp = torch.nn.functional.pad(x[0], (64 - 16, 0))
    spec = torch.stft(xp, 64, 16, 64, torch.hann_window(64), center=False, return_complex=True).abs()[0]
    ref = torch.log((ms.mel_basis @ spec).clamp(1e-5, 1e10))
    assert got.shape == ref.shape and (got - ref).abs().max() < 1e-3
