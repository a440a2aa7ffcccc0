"""VAE families beyond the LDM autoencoder: Klein / FLUX.2 (packed latents + BatchNorm), diffusers key layout (Z-Image),
Wan2.1-style causal 3-D VAE (Qwen-Image) and the Wan2.2 high-compression VAE."""
import pytest
import torch

from mojodiffusion_b200.models import vae as V
from mojodiffusion_b200.models import wan_vae as W


def test_klein_pack_order_and_batchnorm_round_trip():
    z = torch.arange(2 * 3 * 4 * 6, dtype=torch.float32).reshape(2, 3, 4, 6)
    zp = V.KleinVAE.pack(z)
    assert zp.shape == (2, 12, 2, 3)
    c, dy, dx, y, x = 2, 1, 0, 1, 2
    assert zp[1, (c * 2 + dy) * 2 + dx, y, x] == z[1, c, 2 * y + dy, 2 * x + dx]        # packed channel = (c*2+dy)*2+dx
    assert torch.equal(V.KleinVAE.unpack(zp), z)
    cfg = V.VAEConfig(z_channels=4, ch=32, ch_mult=(1, 2), num_res_blocks=1, scale_factor=1.0, shift_factor=0.0, name="tiny-klein-vae")
    vae = V.KleinVAE(cfg, dtype=torch.float32)
    with torch.no_grad():
        vae.init_weights(0)
        vae.bn.running_mean.copy_(torch.linspace(-1, 1, 16))
        vae.bn.running_var.copy_(torch.linspace(0.5, 2.0, 16))
        img = torch.rand(1, 3, 16, 16) * 2 - 1
        lat = vae.encode(img)
        assert lat.shape == (1, 16, 4, 4) and vae.spatial_factor == 4
        out = vae.decode(lat)
        assert out.shape == img.shape and torch.isfinite(out).all()
        # the BatchNorm of encode and its inverse in decode cancel exactly
        mom = vae.quant_conv(vae.encoder(img.permute(0, 2, 3, 1))).float()
        zp = V.KleinVAE.pack(mom[..., :4].permute(0, 3, 1, 2))
        back = lat * torch.sqrt(vae.bn.running_var + 1e-4).view(1, -1, 1, 1) + vae.bn.running_mean.view(1, -1, 1, 1)
        assert torch.allclose(back, zp, atol=1e-5)
    keys = set(vae.state_dict())
    assert {"bn.running_mean", "bn.running_var", "post_quant_conv.weight", "quant_conv.bias"} <= keys


def test_diffusers_key_remap_loads_into_the_ldm_layout():
    cfg = V.tiny_vae_config()
    vae = V.AutoencoderKL(cfg, dtype=torch.float32)
    with torch.no_grad():
        vae.init_weights(1)
    sd = vae.state_dict()
    n = len(cfg.ch_mult)
    # spell the same tensors the diffusers way, then map back
    def to_diffusers(k, v):
        import re
        side, rest = k.split(".", 1)
        rest = rest.replace("nin_shortcut.", "conv_shortcut.")
        if (m := re.match(r"up\.(\d+)\.block\.(\d+)\.(.*)", rest)):
            rest = f"up_blocks.{n - 1 - int(m.group(1))}.resnets.{m.group(2)}.{m.group(3)}"
        elif (m := re.match(r"up\.(\d+)\.upsample\.(.*)", rest)):
            rest = f"up_blocks.{n - 1 - int(m.group(1))}.upsamplers.0.{m.group(2)}"
        elif (m := re.match(r"down\.(\d+)\.block\.(\d+)\.(.*)", rest)):
            rest = f"down_blocks.{m.group(1)}.resnets.{m.group(2)}.{m.group(3)}"
        elif (m := re.match(r"down\.(\d+)\.downsample\.(.*)", rest)):
            rest = f"down_blocks.{m.group(1)}.downsamplers.0.{m.group(2)}"
        elif (m := re.match(r"mid\.block_(\d)\.(.*)", rest)):
            rest = f"mid_block.resnets.{int(m.group(1)) - 1}.{m.group(2)}"
        elif (m := re.match(r"mid\.attn_1\.(\w+)\.(weight|bias)", rest)):
            leaf = {"norm": "group_norm", "q": "to_q", "k": "to_k", "v": "to_v", "proj_out": "to_out.0"}[m.group(1)]
            rest = f"mid_block.attentions.0.{leaf}.{m.group(2)}"
            if m.group(2) == "weight" and v.dim() == 4:
                v = v[:, :, 0, 0]
        elif rest.startswith("norm_out."):
            rest = "conv_norm_out." + rest[len("norm_out."):]
        return f"{side}.{rest}", v
    diff = dict(to_diffusers(k, v) for k, v in sd.items())
    assert "decoder.up_blocks.0.resnets.0.conv1.weight" in diff and "decoder.mid_block.attentions.0.to_q.weight" in diff
    back = V.remap_diffusers_vae_keys(diff, n)
    assert set(back) == set(sd)
    for k in sd:
        assert torch.equal(back[k], sd[k]), k
    assert V.zimage_vae_config().z_channels == 16 and abs(V.zimage_vae_config().scale_factor - 0.3611) < 1e-9


@pytest.mark.parametrize("variant", ["wan21", "wan22"])
def test_wan_vae_shapes_causality_and_image_mode(variant):
    cfg = W.tiny_wan_vae_config(variant)
    vae = W.WanVAE(cfg).init_weights(0)
    f, tf = cfg.spatial_factor, cfg.temporal_factor
    z = torch.randn(1, cfg.z_dim, 3, 4, 4, generator=torch.Generator().manual_seed(0))
    video = vae.decode(z)
    assert video.shape == (1, 3, 1 + tf * 2, 4 * f, 4 * f) and video.abs().max() <= 1.0
    image = vae.decode(z[:, :, 0])
    assert image.shape == (1, 3, 4 * f, 4 * f)
    assert torch.allclose(image, video[:, :, 0], atol=1e-5)              # a single latent frame decodes like the first frame
    z2 = z.clone()
    z2[:, :, 1:] += 1.0
    v2 = vae.decode(z2)
    assert torch.equal(v2[:, :, :1], video[:, :, :1]) and not torch.equal(v2, video)     # causal in time
    x = torch.rand(1, 3, 1 + tf * 2, 4 * f, 4 * f) * 2 - 1
    lat = vae.encode(x)
    assert lat.shape == (1, cfg.z_dim, 3, 4, 4)
    assert vae.encode(x[:, :, 0]).shape == (1, cfg.z_dim, 4, 4)
    x2 = x.clone()
    x2[:, :, 1:] = 0.0
    assert torch.allclose(vae.encode(x2)[:, :, :1], lat[:, :, :1], atol=1e-5)


def test_wan_shortcuts_and_patches_are_inverse_layouts():
    x = torch.randn(1, 4, 4, 6, 6)
    up = W.dup_up3d(x, 2, 2, 2, first_chunk=False)                        # 4 -> 2 channels x (2, 2, 2): 4 copies each
    assert up.shape == (1, 2, 8, 12, 12)
    down = W.avg_down3d(up, 4, 2, 2)
    assert down.shape == x.shape and torch.allclose(down, x, atol=1e-6)   # averaging the duplicates returns the input
    assert W.dup_up3d(x, 2, 2, 2, first_chunk=True).shape[2] == 7
    img = torch.randn(1, 3, 2, 8, 8)
    assert torch.equal(W.unpatchify(W.patchify(img, 2), 2), img)
    assert W.patchify(img, 2).shape == (1, 12, 2, 4, 4)


def test_wan_diffusers_key_remap_and_full_size_structure():
    full = W.WanVAE(W.qwen_image_vae_config(), with_encoder=True)
    keys = set(full.state_dict())
    assert len(full.decoder.upsamples) == 15 and len(full.encoder.downsamples) == 11
    assert full.decoder.conv1.weight.shape == (384, 16, 3, 3, 3) and full.decoder.head[2].weight.shape[0] == 3
    diff = {"decoder.conv_in.weight": 0, "decoder.mid_block.resnets.1.norm2.gamma": 0, "decoder.mid_block.attentions.0.to_qkv.weight": 0,
            "decoder.up_blocks.1.resnets.0.conv_shortcut.weight": 0, "decoder.up_blocks.0.upsamplers.0.time_conv.weight": 0,
            "decoder.up_blocks.2.upsamplers.0.resample.1.bias": 0, "decoder.norm_out.gamma": 0, "decoder.conv_out.bias": 0,
            "encoder.down_blocks.2.resample.1.weight": 0, "encoder.down_blocks.0.conv1.weight": 0, "encoder.down_blocks.3.conv_shortcut.bias": 0,
            "encoder.down_blocks.5.time_conv.weight": 0, "quant_conv.weight": 0, "post_quant_conv.bias": 0}
    mapped = W.remap_diffusers_wan_keys(diff)
    missing = [k for k in mapped if k not in keys]
    assert not missing, missing
    assert "decoder.upsamples.4.shortcut.weight" in mapped and "decoder.upsamples.3.time_conv.weight" in mapped
    w22 = W.wan22_vae_config()
    assert (w22.z_dim, w22.spatial_factor, w22.temporal_factor, len(w22.mean)) == (48, 16, 4, 48)


def test_vae_factory_geometry_and_checkpoint_spellings(tmp_path):
    from mojodiffusion_b200.io.safetensors_io import save_safetensors
    from mojodiffusion_b200.models import vae_factory as F
    cfg = V.VAEConfig(z_channels=4, ch=32, ch_mult=(1, 2), num_res_blocks=1, scale_factor=1.0, shift_factor=0.0)
    klein = V.KleinVAE(cfg, dtype=torch.float32, with_encoder=False)
    assert F.latent_geometry(klein) == (4, 2)
    with torch.no_grad():
        klein.init_weights(0)
        z = torch.randn(1, 4, 4, 4)
        assert F.decode_latent(klein, z).shape == (1, 3, 8, 8)                      # unpacked latent in, packed inside
    wan = W.WanVAE(W.tiny_wan_vae_config("wan21"), with_encoder=False).init_weights(0)
    assert F.latent_geometry(wan) == (4, 4) and F.decode_latent(wan, torch.randn(1, 4, 4, 4)).shape == (1, 3, 16, 16)
    ldm = V.AutoencoderKL(V.tiny_vae_config(), dtype=torch.float32, with_encoder=False)
    with torch.no_grad():
        ldm.init_weights(2)
    sd = {k: v.clone() for k, v in ldm.state_dict().items()}
    spelled = {}
    for k, v in sd.items():                                                        # a few tensors under diffusers names
        k2 = k.replace("decoder.up.1.block.0.", "decoder.up_blocks.0.resnets.0.").replace("decoder.mid.block_1.", "decoder.mid_block.resnets.0.")
        spelled[k2.replace("decoder.norm_out.", "decoder.conv_norm_out.")] = v
    path = str(tmp_path / "vae.safetensors")
    save_safetensors(path, spelled)
    fresh = V.AutoencoderKL(V.tiny_vae_config(), dtype=torch.float32, with_encoder=False)
    assert F.load_vae_weights(fresh, path) == "checkpoint"
    assert torch.equal(fresh.decoder.up[1].block[0].conv1.weight, ldm.decoder.up[1].block[0].conv1.weight)
    assert torch.equal(fresh.decoder.norm_out.weight, ldm.decoder.norm_out.weight)
    assert type(F.build_family_vae("qwenimage", torch.float32, None)).__name__ == "WanVAE"
