"""3-D convolution by temporal taps against torch's conv3d, and the video VAE decoder against a plain-PyTorch statement of
the same schedule (NCDHW, F.conv3d, einops-style rearrangements written out)."""
import torch
import torch.nn.functional as F

from mojodiffusion_b200.models.video_vae import VideoVAE, ltx2_vae_config, tiny_video_vae_config
from mojodiffusion_b200.ops import conv as C


def test_conv3d_by_temporal_taps_matches_torch():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 5, 6, 7, 8, generator=g)
    w = torch.randn(12, 3, 3, 3, 8, generator=g) * 0.1
    b = torch.randn(12, generator=g)
    for pad in ("replicate", "zeros"):
        got = C.conv3d_ndhwc(x, w, b, "silu", pad)
        want = C.conv3d_ndhwc_reference(x, w, b, "silu", pad)
        assert got.shape == (2, 5, 6, 7, 12) and torch.allclose(got, want, atol=1e-4), pad
    one = C.conv3d_ndhwc(x[:, :1], w, b)                       # a single frame sees itself three times
    assert torch.allclose(one, C.conv3d_ndhwc_reference(x[:, :1], w, b), atol=1e-4)


def _plain_decode(sd, cfg, latent):
    def conv(x, name):
        x = F.pad(x, (0, 0, 0, 0, 1, 1), mode="replicate")
        return F.conv3d(x, sd[name + ".conv.weight"], sd[name + ".conv.bias"], padding=(0, 1, 1))

    def pn(x):
        return x * torch.rsqrt(x.pow(2).mean(1, keepdim=True) + 1e-6)

    x = latent * sd["per_channel_statistics.std-of-means"].view(1, -1, 1, 1, 1) + sd["per_channel_statistics.mean-of-means"].view(1, -1, 1, 1, 1)
    h = conv(x, "decoder.conv_in")
    for i, b in enumerate(cfg.blocks):
        p = f"decoder.up_blocks.{i}"
        if b[0] == "mid":
            for r in range(b[2]):
                t = conv(F.silu(pn(h)), f"{p}.res_blocks.{r}.conv1")
                h = h + conv(F.silu(pn(t)), f"{p}.res_blocks.{r}.conv2")
        else:
            ft, fh, fw = b[2:5]
            y = conv(h, p + ".conv")
            B, Cc, T, H, W = y.shape
            c = Cc // (ft * fh * fw)
            y = y.reshape(B, c, ft, fh, fw, T, H, W).permute(0, 1, 5, 2, 6, 3, 7, 4).reshape(B, c, T * ft, H * fh, W * fw)
            h = y[:, :, 1:] if ft == 2 else y
    h = conv(F.silu(pn(h)), "decoder.conv_out")
    B, _, T, H, W = h.shape
    p = cfg.patch
    h = h.reshape(B, cfg.out_channels, p, p, T, H, W).permute(0, 1, 4, 5, 3, 6, 2)
    return h.reshape(B, cfg.out_channels, T, H * p, W * p)


def test_video_vae_decoder_matches_plain_statement():
    cfg = tiny_video_vae_config()
    m = VideoVAE(cfg, torch.float32, "cpu").init_weights(2, std=0.08)
    g = torch.Generator().manual_seed(1)
    getattr(m.per_channel_statistics, "std-of-means").copy_(torch.rand(cfg.latent_channels, generator=g) + 0.5)
    getattr(m.per_channel_statistics, "mean-of-means").copy_(torch.randn(cfg.latent_channels, generator=g) * 0.2)
    z = torch.randn(1, cfg.latent_channels, 3, 4, 5, generator=g)
    got = m.decode(z)
    ft, fs = m.expansion()
    assert (ft, fs) == (2, 8) and got.shape == (1, 3, 1 + (3 - 1) * 2, 4 * 8, 5 * 8)
    want = _plain_decode(m.state_dict(), cfg, z)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-3), float((got - want).abs().max())


def test_ltx2_vae_shape_contract():
    cfg = ltx2_vae_config()
    with torch.device("meta"):
        m = VideoVAE(cfg, torch.bfloat16, "meta")
    assert m.expansion() == (8, 32)                                   # 121 frames at 768x512 <- 16 x 16 x 24 latents
    sd = m.state_dict()
    assert tuple(sd["decoder.conv_in.conv.weight"].shape) == (1024, 128, 3, 3, 3)
    assert tuple(sd["decoder.up_blocks.1.conv.conv.weight"].shape) == (4096, 1024, 3, 3, 3)
    assert tuple(sd["decoder.up_blocks.3.conv.conv.weight"].shape) == (4096, 512, 3, 3, 3)
    assert tuple(sd["decoder.up_blocks.7.conv.conv.weight"].shape) == (512, 256, 3, 3, 3)
    assert tuple(sd["decoder.conv_out.conv.weight"].shape) == (48, 128, 3, 3, 3)
    assert "per_channel_statistics.std-of-means" in sd and "decoder.up_blocks.6.res_blocks.5.conv2.conv.bias" in sd


def _plain_upsample(sd, cfg, z):
    def c3(x, k):
        return F.conv3d(x, sd[k + ".weight"], sd[k + ".bias"], padding=1)

    def gn(x, k):
        return F.group_norm(x, cfg.groups, sd[k + ".weight"], sd[k + ".bias"], eps=1e-5)

    def res(x, p):
        h = F.silu(gn(c3(x, p + ".conv1"), p + ".norm1"))
        return F.silu(gn(c3(h, p + ".conv2"), p + ".norm2") + x)

    x = F.silu(gn(c3(z, "initial_conv"), "initial_norm"))
    for i in range(cfg.blocks):
        x = res(x, f"res_blocks.{i}")
    B, Cc, T, H, W = x.shape
    if cfg.temporal:
        y = c3(x, "upsampler.0")
        y = y.reshape(B, Cc, 2, T, H, W).permute(0, 1, 3, 2, 4, 5).reshape(B, Cc, 2 * T, H, W)
        x = y[:, :, 1:]
    else:
        y = x.permute(0, 2, 1, 3, 4).reshape(B * T, Cc, H, W)
        y = F.pixel_shuffle(F.conv2d(y, sd["upsampler.conv.weight"], sd["upsampler.conv.bias"], padding=1), 2)
        x = y.reshape(B, T, Cc, 2 * H, 2 * W).permute(0, 2, 1, 3, 4)
    for i in range(cfg.blocks):
        x = res(x, f"post_upsample_res_blocks.{i}")
    return c3(x, "final_conv")


def test_latent_upsampler_spatial_and_temporal_match_plain_statement():
    from mojodiffusion_b200.models.latent_upsampler import (LatentUpsampler, ltx2_spatial_upsampler_config,
                                                           ltx2_temporal_upsampler_config, tiny_upsampler_config)
    g = torch.Generator().manual_seed(3)
    for temporal in (False, True):
        cfg = tiny_upsampler_config(temporal)
        m = LatentUpsampler(cfg, torch.float32, "cpu").init_weights(7, std=0.08)
        z = torch.randn(1, cfg.channels, 3, 4, 5, generator=g)
        got = m(z)
        assert got.shape == ((1, cfg.channels, 5, 4, 5) if temporal else (1, cfg.channels, 3, 8, 10))
        want = _plain_upsample(m.state_dict(), cfg, z)
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (temporal, float((got - want).abs().max()))
    with torch.device("meta"):
        sd = LatentUpsampler(ltx2_spatial_upsampler_config(), torch.bfloat16, "meta").state_dict()
        st = LatentUpsampler(ltx2_temporal_upsampler_config(), torch.bfloat16, "meta").state_dict()
    assert tuple(sd["upsampler.conv.weight"].shape) == (4096, 1024, 3, 3) and tuple(sd["initial_conv.weight"].shape) == (1024, 128, 3, 3, 3)
    assert tuple(st["upsampler.0.weight"].shape) == (1024, 512, 3, 3, 3) and "post_upsample_res_blocks.3.norm2.bias" in st


def _plain_encode(sd, cfg, video):
    def conv(x, name):                                     # causal: two copies of the first frame on the left
        x = torch.cat((x[:, :, :1], x[:, :, :1], x), 2)
        return F.conv3d(x, sd[name + ".conv.weight"], sd[name + ".conv.bias"], padding=(0, 1, 1))

    def pn(x, eps=1e-6):
        return x * torch.rsqrt(x.pow(2).mean(1, keepdim=True) + eps)

    def s2d(x, ft, fh, fw):
        B, Cc, T, H, W = x.shape
        x = x.reshape(B, Cc, T // ft, ft, H // fh, fh, W // fw, fw).permute(0, 1, 3, 5, 7, 2, 4, 6)
        return x.reshape(B, Cc * ft * fh * fw, T // ft, H // fh, W // fw)

    B, Cc, T, H, W = video.shape
    p = cfg.patch
    x = video.reshape(B, Cc, T, H // p, p, W // p, p).permute(0, 1, 6, 4, 2, 3, 5).reshape(B, Cc * p * p, T, H // p, W // p)
    h = conv(x, "encoder.conv_in")
    for i, b in enumerate(cfg.enc_blocks):
        pre = f"encoder.down_blocks.{i}"
        if b[0] == "mid":
            for r in range(b[2]):
                t = conv(F.silu(pn(h)), f"{pre}.res_blocks.{r}.conv1")
                h = h + conv(F.silu(pn(t)), f"{pre}.res_blocks.{r}.conv2")
        else:
            cin, cout, ft, fh, fw = b[1:]
            if ft == 2:
                h = torch.cat((h[:, :, :1], h), 2)
            skip = s2d(h, ft, fh, fw)
            g = cin * ft * fh * fw // cout
            if g > 1:
                skip = skip.unflatten(1, (cout, g)).mean(2)
            h = s2d(conv(h, pre + ".conv"), ft, fh, fw) + skip
    h = conv(F.silu(pn(h, 1e-8)), "encoder.conv_out")[:, :cfg.latent_channels]
    return (h - sd["per_channel_statistics.mean-of-means"].view(1, -1, 1, 1, 1)) / sd["per_channel_statistics.std-of-means"].view(1, -1, 1, 1, 1)


def test_video_vae_encoder_matches_plain_statement_and_shapes():
    cfg = tiny_video_vae_config()
    m = VideoVAE(cfg, torch.float32, "cpu", with_encoder=True).init_weights(4, std=0.08)
    g = torch.Generator().manual_seed(2)
    getattr(m.per_channel_statistics, "std-of-means").copy_(torch.rand(cfg.latent_channels, generator=g) + 0.5)
    getattr(m.per_channel_statistics, "mean-of-means").copy_(torch.randn(cfg.latent_channels, generator=g) * 0.2)
    video = torch.randn(1, 3, 5, 16, 24, generator=g)                        # 1 + 2k frames for the tiny 2x temporal factor
    got = m.encode(video)
    assert got.shape == (1, cfg.latent_channels, 3, 2, 3)
    want = _plain_encode(m.state_dict(), cfg, video)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-3), float((got - want).abs().max())
    assert m.decode(got).shape == (1, 3, 5, 16, 24)                            # the decoder inverts the shape
    with torch.device("meta"):
        sd = VideoVAE(ltx2_vae_config(), torch.bfloat16, "meta", with_encoder=True).state_dict()
    assert tuple(sd["encoder.conv_in.conv.weight"].shape) == (128, 48, 3, 3, 3)
    assert tuple(sd["encoder.down_blocks.1.conv.conv.weight"].shape) == (64, 128, 3, 3, 3)
    assert tuple(sd["encoder.down_blocks.5.conv.conv.weight"].shape) == (128, 512, 3, 3, 3)
    assert tuple(sd["encoder.down_blocks.7.conv.conv.weight"].shape) == (128, 1024, 3, 3, 3)
    assert tuple(sd["encoder.conv_out.conv.weight"].shape) == (129, 1024, 3, 3, 3)
