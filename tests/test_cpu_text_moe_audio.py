"""Text encoders against the Hugging Face implementations (tiny random configs, same weights), tokenizers on synthetic
vocabularies, MoE primitives against a per-token loop, audio ops identities."""
import json

import math

import pytest
import torch

from mojodiffusion_b200.models.text import (ByteLevelBPE, CLIPTextConfig, CLIPTextEncoder, CLIPTokenizer, Qwen3Config, Qwen3Encoder,
                                            T5Config, T5Encoder)
from mojodiffusion_b200.models.text.tokenizers import bytes_to_unicode
from mojodiffusion_b200.models.vocoder import Vocoder, tiny_vocoder_config
from mojodiffusion_b200.ops import audio, moe

transformers = pytest.importorskip("transformers")


def test_clip_text_encoder_matches_hf():
    torch.manual_seed(0)
    hc = transformers.CLIPTextConfig(vocab_size=99, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                                     max_position_embeddings=16, eos_token_id=98, bos_token_id=97, pad_token_id=98)
    hf = transformers.CLIPTextModel(hc).eval()
    mine = CLIPTextEncoder(CLIPTextConfig(99, 32, 64, 3, 4, 16, "quick_gelu", 1e-5, 98))
    missing, unexpected = mine.load_state_dict(hf.state_dict(), strict=False)
    assert not missing and all("position_ids" in u for u in unexpected)
    ids = torch.tensor([[97, 5, 6, 7, 98, 98, 98, 98], [97, 9, 98, 98, 98, 98, 98, 98]])
    with torch.no_grad():
        ref = hf(ids)
    last, pooled = mine(ids)
    assert torch.allclose(last, ref.last_hidden_state, atol=1e-5) and torch.allclose(pooled, ref.pooler_output, atol=1e-5)


def test_t5_encoder_matches_hf():
    torch.manual_seed(0)
    hc = transformers.T5Config(vocab_size=64, d_model=32, d_kv=8, d_ff=48, num_layers=3, num_heads=4, feed_forward_proj="gated-gelu",
                               relative_attention_num_buckets=8, relative_attention_max_distance=16)
    hf = transformers.T5EncoderModel(hc).eval()
    mine = T5Encoder(T5Config(64, 32, 8, 48, 3, 4, 8, 16, 1e-6))
    missing, unexpected = mine.load_state_dict(hf.state_dict(), strict=False)
    assert not missing and all("embed_tokens" in u for u in unexpected)
    ids = torch.randint(2, 64, (2, 11))
    mask = torch.ones(2, 11, dtype=torch.long)
    mask[1, 7:] = 0
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=mask).last_hidden_state
    out = mine(ids, mask)
    assert torch.allclose(out[0], ref[0], atol=2e-5) and torch.allclose(out[1, :7], ref[1, :7], atol=2e-5)


def test_qwen3_encoder_matches_hf():
    if not hasattr(transformers, "Qwen3Model"):
        pytest.skip("transformers without Qwen3")
    torch.manual_seed(0)
    hc = transformers.Qwen3Config(vocab_size=80, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                                  num_key_value_heads=2, head_dim=8, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=64)
    hf = transformers.Qwen3Model(hc).eval()
    mine = Qwen3Encoder(Qwen3Config(80, 32, 64, 3, 4, 2, 8, 1e-6, 10000.0))
    sd = {"model." + k: v for k, v in hf.state_dict().items()}
    missing, unexpected = mine.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    ids = torch.randint(0, 80, (2, 9))
    with torch.no_grad():
        ref = hf(input_ids=ids, output_hidden_states=True)
    assert torch.allclose(mine(ids), ref.last_hidden_state, atol=2e-5)
    assert torch.allclose(mine(ids, layer=-2, final_norm=False), ref.hidden_states[-2], atol=2e-5)


def test_mistral_style_encoder_matches_hf_and_scaled_rotary_frequencies():
    """The decoder stack without QK norms equals transformers' MistralModel (hidden state of a middle layer included); the scaled
    inverse frequencies follow the three-band rule, and with the ERNIE encoder's constants every frequency is divided by 16."""
    import math
    from mojodiffusion_b200.models.text import qwen3 as Q
    if not hasattr(transformers, "MistralModel"):
        pytest.skip("transformers without Mistral")
    torch.manual_seed(0)
    hc = transformers.MistralConfig(vocab_size=80, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4,
                                    num_key_value_heads=2, head_dim=8, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=64,
                                    sliding_window=None)
    hf = transformers.MistralModel(hc).eval()
    mine = Qwen3Encoder(Qwen3Config(80, 32, 64, 4, 4, 2, 8, 1e-5, 10000.0, qk_norm=False))
    raw = {"language_model.model." + k: v for k, v in hf.state_dict().items()}
    raw["vision_tower.x"] = torch.zeros(1)
    missing, unexpected = mine.load_state_dict(Q.remap_mistral3b_keys(raw), strict=False)
    assert not missing and not unexpected
    ids, real = Q.pad_or_trim_ids([1, 5, 9, 33, 7], 9)
    assert ids == [1, 5, 9, 33, 7, 0, 0, 0, 0] and real == 5 and Q.pad_or_trim_ids(range(20), 4) == ([0, 1, 2, 3], 4)
    t = torch.tensor([ids])
    with torch.no_grad():
        ref = hf(input_ids=t, output_hidden_states=True)
    assert torch.allclose(mine(t, layer=3, final_norm=False), ref.hidden_states[3], atol=2e-5)
    assert torch.allclose(mine(t), ref.last_hidden_state, atol=2e-5)

    c = Q.mistral3b_config()
    assert (c.num_hidden_layers, c.hidden_size, c.num_key_value_heads, Q.MISTRAL3B_EXTRACT_LAYER) == (26, 3072, 8, 24) and not c.qk_norm
    base = 1.0 / (1.0e6 ** (torch.arange(0, 128, 2, dtype=torch.float64) / 128))
    assert torch.allclose(Q.scaled_inv_freq(128, 1.0e6, c.rope_scaling).double(), base / 16.0, rtol=1e-6)
    assert torch.allclose(Q.scaled_inv_freq(128, 1.0e6, None).double(), base, rtol=1e-6)
    # a setting that exercises all three bands: orig 64 positions, beta_fast 4 -> low 41, beta_slow 0.2 -> high 2
    got = Q.scaled_inv_freq(16, 100.0, (8.0, 64, 4.0, 0.2)).double()
    low, high = float(int(64 / (2 * math.pi / 4.0) + 0.5)), float(int(64 / (2 * math.pi / 0.2) + 0.5))
    for i in range(8):
        f = 1.0 / 100.0 ** (2 * i / 16)
        wl = 2 * math.pi / f
        if wl < 64 / high:
            want = f
        elif wl > 64 / low:
            want = f / 8.0
        else:
            sm = (64 / wl - low) / (high - low)
            want = (1 - sm) * f / 8.0 + sm * f
        assert abs(float(got[i]) - want) < 1e-7 * max(1.0, want)


def test_qwen25vl_language_stack_matches_hf_qwen2():
    """Biased q / k / v projections without QK norms: the Qwen2.5-VL language stack equals transformers' Qwen2Model."""
    from mojodiffusion_b200.models.text import qwen3 as Q
    if not hasattr(transformers, "Qwen2Model"):
        pytest.skip("transformers without Qwen2")
    torch.manual_seed(2)
    hc = transformers.Qwen2Config(vocab_size=80, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                                  num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=1.0e6, max_position_embeddings=64, use_sliding_window=False)
    hf = transformers.Qwen2Model(hc).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("_proj.bias"):
                p.normal_(0, 0.1)
    mine = Qwen3Encoder(Qwen3Config(80, 32, 64, 3, 4, 2, 8, 1e-6, 1.0e6, qk_norm=False, qkv_bias=True))
    missing, unexpected = mine.load_state_dict(Q.remap_qwen3vl_text_keys({"model.language_model." + k: v for k, v in hf.state_dict().items()}, torch.float32), strict=False)
    assert not missing and not unexpected
    ids = torch.randint(0, 80, (2, 11))
    with torch.no_grad():
        ref = hf(input_ids=ids, output_hidden_states=True)
    assert torch.allclose(mine(ids), ref.last_hidden_state, atol=3e-5) and torch.allclose(mine.layer_states(ids)[1], ref.hidden_states[2], atol=3e-5)
    c = Q.qwen25vl_text_config()
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.intermediate_size) == (28, 3584, 28, 4, 18944)
    full = Qwen3Encoder(c, torch.float32, "meta").state_dict()
    assert full["model.layers.0.self_attn.k_proj.bias"].shape == (512,) and "model.layers.0.self_attn.o_proj.bias" not in full and "model.layers.0.self_attn.q_norm.weight" not in full


def test_gpt_oss_encoder_matches_hf_and_mxfp4_expert_mapping():
    """Sinks, alternating sliding-window / full causal layers, YaRN rotary scaling and the clamped interleaved mixture equal
    transformers' GptOssModel; packed e2m1 + e8m0 expert tensors map onto the dense layout."""
    from mojodiffusion_b200.models.text import gpt_oss as G
    if not hasattr(transformers, "GptOssModel"):
        pytest.skip("transformers without GPT-OSS")
    torch.manual_seed(3)
    rope = {"rope_type": "yarn", "factor": 32.0, "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False,
            "original_max_position_embeddings": 4096, "rope_theta": 150000.0}
    try:
        hc = transformers.GptOssConfig(vocab_size=90, hidden_size=32, intermediate_size=24, num_hidden_layers=4, num_attention_heads=4,
                                       num_key_value_heads=2, head_dim=16, num_local_experts=6, num_experts_per_tok=2, sliding_window=4,
                                       rms_norm_eps=1e-5, max_position_embeddings=8192, rope_parameters=rope, attention_bias=True)
    except TypeError:
        pytest.skip("GptOssConfig signature differs")
    hc._attn_implementation = "eager"
    hf = transformers.GptOssModel(hc).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("sinks") or n.endswith("bias"):
                p.normal_(0, 0.3)
            elif "experts" in n or "router" in n:
                p.normal_(0, 0.2)
    assert [hc.layer_types[i] for i in range(4)] == ["sliding_attention", "full_attention"] * 2
    cfg = G.GptOssConfig(vocab_size=90, hidden_size=32, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                         intermediate_size=24, num_local_experts=6, num_experts_per_tok=2, sliding_window=4)
    mine = G.GptOssEncoder(cfg)
    missing, unexpected = mine.load_state_dict(G.remap_gpt_oss_keys({"model." + k: v for k, v in hf.state_dict().items()}), strict=False)
    assert not missing and not unexpected
    ids = torch.randint(0, 90, (2, 13))
    with torch.no_grad():
        ref = hf(input_ids=ids, output_hidden_states=True)
    st = mine.layer_states(ids)
    for i in range(4):
        assert torch.allclose(st[i], ref.hidden_states[i + 1] if i < 3 else st[i], atol=1e-4), i
    assert torch.allclose(mine(ids), ref.last_hidden_state, atol=1e-4)
    feats = mine.lens_features(ids, layers=(0, 2))
    assert feats.shape == (2, 13, 2, 32) and torch.equal(feats[:, :, 1], st[2])
    full = G.GptOssConfig()
    inv, mult = G.yarn_inv_freq(full)
    assert inv.shape == (32,) and abs(mult - (0.1 * math.log(32.0) + 1.0)) < 1e-12 and abs(float(inv[0]) - 1.0) < 1e-6
    assert abs(float(inv[-1]) - 1.0 / (32.0 * 150000.0 ** (62 / 64))) < 1e-12 and G.LENS_CAPTURE_LAYERS == (5, 11, 17, 23)
    # packed experts: [experts, out, G, 16] blocks + [experts, out, G] scales
    E, out_f, Gn = 2, 3, 2
    blocks = torch.randint(0, 256, (E, out_f, Gn, 16), dtype=torch.uint8)
    scales = torch.randint(125, 130, (E, out_f, Gn), dtype=torch.uint8)
    dense = G.dequant_mxfp4(blocks, scales, torch.float32)
    assert dense.shape == (E, out_f, Gn * 32)
    e, o, g, b = 1, 2, 1, 5
    byte = int(blocks[e, o, g, b])
    sc = 2.0 ** (int(scales[e, o, g]) - 127)
    assert float(dense[e, o, g * 32 + 2 * b]) == G._FP4[byte & 15] * sc and float(dense[e, o, g * 32 + 2 * b + 1]) == G._FP4[byte >> 4] * sc
    m = G.remap_gpt_oss_keys({"model.layers.0.mlp.experts.down_proj_blocks": blocks, "model.layers.0.mlp.experts.down_proj_scales": scales,
                              "model.norm.weight": torch.ones(2), "lm_head.weight": torch.ones(2)}, torch.float32)
    assert set(m) == {"layers.0.mlp.experts.down_proj", "norm.weight"} and torch.equal(m["layers.0.mlp.experts.down_proj"], dense.transpose(1, 2))


def test_qwen3vl_text_paths_layer_stacks_and_key_mapping():
    """Layer outputs equal transformers' hidden_states; Krea-2 stacks twelve of them and drops the template rows; Ideogram-4
    interleaves thirteen taps per feature; checkpoint prefixes and fp8 rows map onto the encoder's names."""
    from mojodiffusion_b200.models.text import qwen3 as Q
    if not hasattr(transformers, "Qwen3Model"):
        pytest.skip("transformers without Qwen3")
    torch.manual_seed(1)
    hc = transformers.Qwen3Config(vocab_size=80, hidden_size=32, intermediate_size=64, num_hidden_layers=36, num_attention_heads=4,
                                  num_key_value_heads=2, head_dim=8, rms_norm_eps=1e-6, rope_theta=5.0e6, max_position_embeddings=128)
    hf = transformers.Qwen3Model(hc).eval()
    mine = Qwen3Encoder(Qwen3Config(80, 32, 64, 36, 4, 2, 8, 1e-6, 5.0e6))
    raw = {"model.language_model." + k: v for k, v in hf.state_dict().items()}
    raw["model.visual.patch_embed.weight"] = torch.zeros(2)
    missing, unexpected = mine.load_state_dict(Q.remap_qwen3vl_text_keys(raw, torch.float32), strict=False)
    assert not missing and not unexpected
    ids = torch.randint(0, 80, (1, 40))
    with torch.no_grad():
        ref = hf(input_ids=ids, output_hidden_states=True).hidden_states
    states = mine.layer_states(ids)
    assert len(states) == 36 and all(torch.allclose(states[i], ref[i + 1], atol=5e-5) for i in (0, 7, 34))
    k = Q.krea2_text_features(mine, ids)
    assert k.shape == (1, 6, 12, 32) and torch.allclose(k[0, :, 3], ref[11][0, 34:], atol=5e-5) and torch.allclose(k[0, :, 11], ref[35][0, 34:], atol=5e-5)
    with pytest.raises(ValueError):
        Q.krea2_text_features(mine, ids[:, :30])
    f = Q.ideogram_text_features(mine, ids)
    assert f.shape == (1, 40, 13 * 32) and torch.allclose(f[0, :, 5 * 13 + 2], ref[7][0, :, 5], atol=5e-5) and torch.allclose(f[0, :, 12], ref[36 - 0][0, :, 0] * 0 + states[35][0, :, 0], atol=5e-5)
    assert torch.allclose(Q.boogu_text_features(mine, ids), hf(input_ids=ids).last_hidden_state, atol=5e-5)
    assert Q.qwen3vl_text_config("4b").hidden_size == 2560 and Q.qwen3vl_text_config().intermediate_size == 12288 and Q.qwen3vl_text_config().rope_theta == 5.0e6
    w8 = torch.randn(4, 8).clamp(-3, 3).to(torch.float8_e4m3fn)
    m = Q.remap_qwen3vl_text_keys({"language_model.layers.0.self_attn.q_proj.weight": w8,
                                   "language_model.layers.0.self_attn.q_proj.weight_scale": torch.tensor([1.0, 2.0, 0.5, 4.0]),
                                   "language_model.norm.weight": torch.ones(3)}, torch.float32)
    assert set(m) == {"model.layers.0.self_attn.q_proj.weight", "model.norm.weight"}
    assert torch.equal(m["model.layers.0.self_attn.q_proj.weight"], w8.float() * torch.tensor([1.0, 2.0, 0.5, 4.0])[:, None])


def test_tokenizers_on_synthetic_vocab(tmp_path):
    b2u = bytes_to_unicode()
    assert len(b2u) == 256 and len(set(b2u.values())) == 256
    base = [b2u[b] for b in range(256)]
    vocab = {}
    for s in base + [c + "</w>" for c in base]:
        vocab.setdefault(s, len(vocab))
    merges = [("c", "a"), ("ca", "t</w>"), ("d", "o"), ("do", "g</w>")]
    for a, b in merges:
        vocab.setdefault(a + b, len(vocab))
    vocab["<|startoftext|>"], vocab["<|endoftext|>"] = len(vocab), len(vocab) + 1
    json.dump(vocab, open(tmp_path / "vocab.json", "w"))
    open(tmp_path / "merges.txt", "w").write("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges) + "\n")
    tok = CLIPTokenizer.from_files(str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt"), max_length=12)
    ids, mask = tok("A  Cat, dog!")
    assert ids[0] == vocab["<|startoftext|>"] and len(ids) == 12 and sum(mask) == 7
    assert vocab["cat</w>"] in ids and vocab["dog</w>"] in ids and ids[sum(mask) - 1] == vocab["<|endoftext|>"]
    assert tok.decode(ids[:sum(mask)]) == "a cat , dog !"
    bv = {s: i for i, s in enumerate(base)}
    bm = [("h", "e"), ("l", "l"), ("he", "ll"), ("Ġ", "w")]
    for a, b in bm:
        bv.setdefault(a + b, len(bv))
    bl = ByteLevelBPE(bv, bm, {"<|im_start|>": 1000, "<|im_end|>": 1001})
    text = "<|im_start|>hello wörld\n<|im_end|>"
    enc = bl.encode(text)
    assert enc[0] == 1000 and enc[-1] == 1001 and bv["hell"] in enc and bv["Ġw"] in enc
    assert bl.decode(enc) == text
    assert "<|im_start|>user\nhi<|im_end|>" in bl.chat_template("hi")


def test_moe_primitives():
    torch.manual_seed(0)
    T, H, E, Fd, k = 37, 16, 4, 24, 2
    x, rw = torch.randn(T, H), torch.randn(E, H)
    gw, uw, dw = torch.randn(E, Fd, H) * 0.2, torch.randn(E, Fd, H) * 0.2, torch.randn(E, H, Fd) * 0.2
    ids, gating = moe.top_k_router(torch.tensor([[1.0, 3.0, 3.0, 0.0]]), 2)
    assert ids.tolist() == [1, 2] and torch.allclose(gating, torch.tensor([0.5, 0.5]))      # tie -> lower expert first
    y = moe.moe_ffn(x, rw, gw, uw, dw, k)
    top = (x @ rw.T).topk(k, dim=1)
    g = torch.softmax(top.values, 1)
    ref = torch.zeros_like(x)
    for t in range(T):
        for j in range(k):
            e = int(top.indices[t, j])
            ref[t] += g[t, j] * ((torch.nn.functional.silu(x[t] @ gw[e].T) * (x[t] @ uw[e].T)) @ dw[e].T)
    assert torch.allclose(y, ref, atol=1e-5)
    acc = torch.zeros(3, 2)
    moe.gated_scatter_add(torch.ones(4, 2), torch.tensor([1.0, 2.0, 3.0, 4.0]), torch.tensor([0, 0, 2, 7]), acc)
    assert acc.tolist() == [[3.0, 3.0], [0.0, 0.0], [3.0, 3.0]]


def test_audio_ops_and_vocoder():
    torch.manual_seed(0)
    x, w = torch.randn(2, 8, 50), torch.randn(8, 4, 5)
    a = audio.conv_transpose1d(x, w, None, stride=3, padding=1)
    b = audio.conv_transpose1d(x, w, None, stride=3, padding=1, zero_insert=True)
    assert a.shape == b.shape == (2, 4, 150) and torch.allclose(a, b, atol=1e-4)
    assert audio.zero_insert1d(torch.ones(1, 1, 3), 2).flatten().tolist() == [1, 0, 1, 0, 1]
    assert audio.replicate_pad1d(torch.tensor([[[1.0, 2.0]]]), 2, 1).flatten().tolist() == [1, 1, 1, 2, 2]
    sig = torch.randn(1, 1024)
    m, p = audio.stft(sig, 64, 16)
    assert torch.allclose(audio.istft(m, p, 64, 16, length=1024), sig, atol=1e-4)
    fb = audio.mel_filterbank(10, 64, 16000)
    assert fb.shape == (10, 33) and (fb >= 0).all() and (fb.sum(1) > 0).all()
    assert audio.log_mel(sig, 64, 16, 10, 16000).shape[1] == 10
    s = audio.snake(torch.tensor([[[0.5]]]), torch.zeros(1), None)
    assert abs(float(s) - (0.5 + torch.sin(torch.tensor(0.5)) ** 2)) < 1e-6
    v = Vocoder(tiny_vocoder_config())
    wav = v(torch.randn(1, 16, 10))
    assert wav.shape == (1, 10 * v.hop) and wav.abs().max() <= 1.0
    import dataclasses
    v2 = Vocoder(dataclasses.replace(tiny_vocoder_config(), istft_head=True))
    assert v2(torch.randn(1, 16, 10)).dim() == 2


def test_mx_block_formats_reference():
    """MXFP4 / MXFP8: known encodings decode to their values, quantise -> dequantise -> quantise is stable, the error stays
    inside the format's bound, and the gpt-oss tensor layout ([.., G, 16] blocks + [.., G] scales) reshapes to [.., G * 32]."""
    import torch
    from mojodiffusion_b200 import ops as O
    blocks = torch.zeros(1, 16, dtype=torch.uint8)
    blocks[0, 0] = 0x21            # low nibble 1 -> 0.5, high nibble 2 -> 1.0
    blocks[0, 1] = 0xF7            # low nibble 7 -> 6.0, high nibble 15 -> -6.0
    y = O.mx_dequant(blocks, torch.tensor([128], dtype=torch.uint8)).float()       # scale 2^1
    assert y[:4].tolist() == [1.0, 2.0, 12.0, -12.0] and float(y[4:].abs().max()) == 0.0
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(64, 64, generator=g) * torch.logspace(-3, 3, 64)[:, None]).bfloat16()
    for fp4, bound in ((True, 0.26), (False, 0.13)):
        q, s = O.mx_quant(x, fp4)
        assert q.dtype == torch.uint8 and s.numel() == x.numel() // 32 and q.numel() == x.numel() // (2 if fp4 else 1)
        back = O.mx_dequant(q, s, fp4).reshape(x.shape)
        blk = x.float().reshape(-1, 32)
        err = (back.float().reshape(-1, 32) - blk).abs().amax(dim=1) / blk.abs().amax(dim=1)
        assert float(err.max()) < bound
        q2, s2 = O.mx_quant(back, fp4)
        assert torch.equal(q2, q) and torch.equal(s2, s)
    z, sz = O.mx_quant(torch.zeros(64, dtype=torch.bfloat16), True)
    assert int(sz.max()) == 0 and int(z.max()) == 0
    w = O.mx_dequant(torch.randint(0, 256, (3, 5, 4, 16), dtype=torch.uint8, generator=g), torch.randint(110, 130, (3, 5, 4), dtype=torch.uint8, generator=g))
    assert w.shape == (3, 5, 128) and w.dtype == torch.bfloat16


def test_mxfp8_operand_layout_and_reference_product():
    """The scale chunks of the block-scaled GEMM: byte (r % 32) * 16 + (r % 128 // 32) * 4 + k32 % 4 of chunk
    (r // 128, k32 // 4), padding bytes 127; the dequantised product stays within the format's error of the bf16 product."""
    import torch
    from mojodiffusion_b200 import ops as O
    from mojodiffusion_b200.ops import reference as R
    g = torch.Generator().manual_seed(0)
    x = torch.randn(200, 256, generator=g).bfloat16()
    w = (torch.randn(264, 256, generator=g) * 0.05).bfloat16()
    xq, xs = O.mxfp8_quant_rows(x, 128)
    wq, ws = O.mxfp8_quant_rows(w, 256)
    assert xq.shape == (200, 256) and xs.shape == (2, 2, 512) and ws.shape == (4, 2, 512)
    _, e = O.mx_quant(x, fp4=False)
    e = e.reshape(200, 8)
    r, k = 133, 5
    assert xs[r // 128, k // 4, (r % 32) * 16 + (r % 128 // 32) * 4 + k % 4] == e[r, k]
    assert torch.equal(R.mxfp8_scales_from_chunks(xs, 200, 256), e)
    assert int(xs[1, 0, (200 % 32) * 16 + (200 % 128 // 32) * 4]) == 127          # rows past the end keep the neutral scale
    y = O.gemm_mxfp8(xq, xs, wq, ws)
    want = x.float() @ w.float().t()
    cos = torch.nn.functional.cosine_similarity(y.float().flatten(), want.flatten(), dim=0)
    assert y.shape == (200, 264) and float(cos) > 0.998
    lin = O.MXFP8Weight(w, torch.zeros(264).bfloat16())
    assert torch.equal(lin.linear(x.reshape(2, 100, 256)).reshape(200, 264), y)
