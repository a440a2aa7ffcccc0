"""CPU tests: cap-cache bins, PNG / WAV, run configs and sample-prompt files."""
import glob
import json
import os

import numpy as np
import pytest
import torch

from mojodiffusion_b200 import io as mio


def test_cap_cache_bit_exact(tmp_path):
    for t in (torch.randn(3, 77, 16).bfloat16(), torch.randn(5).float(), torch.arange(6, dtype=torch.int64).reshape(2, 3),
              torch.randn(4, 8).to(torch.float8_e4m3fn)):
        p = tmp_path / "t.bin"
        mio.save_tensor_bin(p, t)
        back = mio.load_tensor_bin(p)
        assert back.dtype == t.dtype and back.shape == t.shape
        assert torch.equal(back.view(torch.uint8), t.contiguous().view(torch.uint8))
    raw = bytearray((tmp_path / "t.bin").read_bytes())
    raw[0] ^= 1
    (tmp_path / "bad.bin").write_bytes(raw)
    with pytest.raises(ValueError):
        mio.load_tensor_bin(tmp_path / "bad.bin")
    (tmp_path / "short.bin").write_bytes(bytes(raw[:-3]))
    with pytest.raises(ValueError):
        mio.load_tensor_bin(tmp_path / "short.bin")


def test_png_roundtrip_with_text(tmp_path):
    rng = np.random.default_rng(0)
    for c in (1, 3, 4):
        img = rng.integers(0, 256, size=(13, 17, c), dtype=np.uint8)
        p = tmp_path / f"a{c}.png"
        mio.save_png(p, img if c > 1 else img[:, :, 0], {"serenity.genparams.v1": json.dumps({"seed": 42, "steps": 28})})
        back, text = mio.load_png(p)
        assert np.array_equal(back, img)
        assert json.loads(text["serenity.genparams.v1"])["seed"] == 42
        assert p.read_bytes()[:8] == b"\x89PNG\r\n\x1a\n"
    x = torch.linspace(-1, 1, 3 * 4 * 5).reshape(3, 4, 5)
    u = mio.tensor_to_uint8(x)
    assert u.shape == (4, 5, 3) and int(u.min()) == 0 and int(u.max()) == 255


def test_wav_header(tmp_path):
    t = torch.sin(torch.linspace(0, 20, 1000))
    mio.save_wav(tmp_path / "a.wav", torch.stack([t, -t], 1), 16000)
    b = (tmp_path / "a.wav").read_bytes()
    assert b[:4] == b"RIFF" and b[8:12] == b"WAVE" and len(b) == 44 + 1000 * 2 * 2
    assert int.from_bytes(b[24:28], "little") == 16000 and int.from_bytes(b[22:24], "little") == 2


def test_every_packaged_config_loads():
    here = os.path.join(os.path.dirname(mio.__file__), "..", "configs")
    files = sorted(glob.glob(os.path.join(here, "*.json")))
    assert len(files) >= 5
    for f in files:
        d = json.load(open(f))
        if d.get("schema"):
            sp = mio.read_sample_prompts(f)
            assert sp.prompts and sp.by_id(sp.prompts[0].id).steps > 0
            continue
        cfg = mio.read_model_config(f)
        assert cfg.model_type and not cfg.extra, (f, cfg.extra)
    cfg = mio.read_model_config({"model_type": "flux", "learning_rate": 3e-4, "lr_scheduler": "cosine", "lr_warmup_steps": 200,
                                 "optimizer": {"eps": 1e-8, "weight_decay": 0.02, "beta1": 0.9, "beta2": 0.99},
                                 "_comment_lora": "x", "some_future_key": 5})
    assert cfg.optimizer.weight_decay == 0.02 and cfg.scheduler_name == "cosine" and cfg.warmup_steps == 200
    assert cfg.extra == {"some_future_key": 5} and cfg.max_steps == 3000 and cfg.save_every == 500 and cfg.sample_every == 250


def test_reference_config_key_set_is_covered():
    # every key that appears in the reference's 35 config files (collected once, listed here as text)
    keys = """adm_in_channels algo base_model_name batch_size beta_end beta_start cache_dir caption_dropout_prob channel_mult
    checkpoint concept_file_name context_dim controlnet_layers controlnet_scale dataset_cache_dir dataset_path ema ema_decay
    ema_min_decay ema_update_after_step ema_update_step_interval embedding_weight_dtype enable_activation_offloading
    enable_async_offloading fallback_train_dtype final_norm_eps gradient_checkpointing head_dim huber_delta in_channels
    init_lokr_norm inner_dim joint_attention_dim layer_offload_fraction learning_rate learning_rate_scheduler
    learning_rate_warmup_steps lokr_decompose_both lokr_factor lokr_factor_attn lokr_factor_ff lokr_factor_single
    lokr_full_matrix lokr_targets lora_alpha lora_rank lora_weight_dtype loss_fn lr_scheduler lr_warmup_steps max_grad_norm
    max_steps min_mod min_snr_gamma_flow mlp_hidden model_channels model_type non_ema_sampling norm_eps num_context_refiner
    num_double num_groups num_heads num_noise_refiner num_res_blocks num_single num_train_timesteps optimizer out_channels
    output_dtype output_model_destination output_model_format pad_tokens_multiple patch_size prediction_type
    quantized_resident resolution rope_axes_dim rope_theta sample_after sample_after_unit sample_at_start
    sample_definition_file_name sample_every sample_shift sample_skip_first save_before_sample save_every save_every_unit
    save_skip_first seed smooth_l1_beta stop_training_after stop_training_after_unit text_encoder text_encoder_2
    text_encoder_weight_dtype time_embed_dim time_scale timestep_dim timestep_distribution timestep_noising_bias
    timestep_noising_weight timestep_shift train_dtype train_num_steps training_method transformer_depth_input
    transformer_depth_middle transformer_depth_output transformer_weight_dtype trigger_word vae vae_weight_dtype
    validation_prompts_file weight_dtype workspace_dir""".split()
    from dataclasses import fields
    have = {f.name for f in fields(mio.TrainConfig)}
    assert not [k for k in keys if k not in have]


def test_disk_guard(tmp_path):
    mio.guard_free_space(tmp_path / "x" / "y.safetensors", 1024)
    with pytest.raises(OSError):
        mio.guard_free_space(tmp_path, 1 << 60)
