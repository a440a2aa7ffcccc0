"""KV-cached decode equals a full re-run of the stack at every step; the sampler's generator, filters and edge cases."""
import torch

from mojodiffusion_b200.llm import KVCache, Qwen3Decoder, Rng, SamplerConfig, argmax, sample, single_query_attention
from mojodiffusion_b200.models.text.qwen3 import Qwen3Config, Qwen3Encoder


def _tiny():
    torch.manual_seed(0)
    cfg = Qwen3Config(vocab_size=97, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, rope_theta=10000.0)
    return cfg, Qwen3Encoder(cfg, torch.float32, "cpu")


def test_incremental_decode_matches_full_forward():
    cfg, enc = _tiny()
    dec = Qwen3Decoder(enc)
    ids = torch.tensor([[5, 17, 3, 88, 42, 9]])
    hidden, cache = dec.prefill(ids[:, :3], max_len=8)
    assert cache.length == 3
    full = enc(ids[:, :3], final_norm=False)
    assert torch.allclose(hidden, full[:, -1], atol=1e-5)
    for t in range(3, 6):
        hidden = dec.decode_step(ids[:, t], cache)
        full = enc(ids[:, :t + 1], final_norm=False)
        assert torch.allclose(hidden, full[:, -1], atol=2e-5), t
    assert cache.length == 6
    lg = dec.logits(hidden)
    assert lg.shape == (1, cfg.vocab_size)
    want = enc(ids)[:, -1].float() @ enc.model.embed_tokens.weight.float().t()
    assert torch.allclose(lg, want, atol=1e-4)


def test_single_query_attention_grouping():
    g = torch.Generator().manual_seed(1)
    B, H, Hkv, T, Dh = 2, 6, 2, 7, 8
    q, k, v = torch.randn(B, H, Dh, generator=g), torch.randn(B, Hkv, T, Dh, generator=g), torch.randn(B, Hkv, T, Dh, generator=g)
    got = single_query_attention(q, k, v, 5)
    kk, vv = k[:, :, :5].repeat_interleave(3, 1), v[:, :, :5].repeat_interleave(3, 1)
    want = torch.softmax((q[:, :, None] * kk).sum(-1) * Dh ** -0.5, -1)[..., None].mul(vv).sum(2)
    assert torch.allclose(got, want, atol=1e-5)


def test_generate_is_deterministic_and_stops_at_eos():
    cfg, enc = _tiny()
    dec = Qwen3Decoder(enc)
    a = dec.generate([1, 2, 3], 6, SamplerConfig(temperature=0.8, top_k=20, top_p=0.9, seed=7))
    b = dec.generate([1, 2, 3], 6, SamplerConfig(temperature=0.8, top_k=20, top_p=0.9, seed=7))
    assert a == b and len(a) == 6
    greedy = dec.generate([1, 2, 3], 4, SamplerConfig(temperature=0.0))
    stop = dec.generate([1, 2, 3], 4, SamplerConfig(temperature=0.0), eos_ids=(greedy[1],))
    assert stop == greedy[:greedy.index(greedy[1]) + 1]


def test_rng_is_xorshift64star_with_53_bit_uniform():
    r = Rng(1)
    x = 1
    x ^= x >> 12
    x ^= (x << 25) & (2 ** 64 - 1)
    x ^= x >> 27
    assert r.next_u64() == (x * 0x2545F4914F6CDD1D) % 2 ** 64
    assert Rng(0).state == 0x9E3779B97F4A7C15
    r = Rng(123)
    u = [r.next_f64() for _ in range(4000)]
    assert 0.0 <= min(u) and max(u) < 1.0 and max(u) > 0.9 and 0.47 < sum(u) / len(u) < 0.53


def test_sampler_filters():
    logits = [0.0, 3.0, 1.0, 3.0, -2.0]
    assert argmax(logits) == 1                                             # first of the tied maxima
    assert sample(logits, SamplerConfig(temperature=0.0), Rng(1)) == 1
    r = Rng(5)
    assert all(sample(logits, SamplerConfig(temperature=1.0, top_k=1), r) == 1 for _ in range(20))
    r = Rng(6)
    picks = {sample(logits, SamplerConfig(temperature=1.0, top_k=2), r) for _ in range(200)}
    assert picks == {1, 3}
    r = Rng(7)
    picks = {sample(logits, SamplerConfig(temperature=1.0, top_p=0.5), r) for _ in range(200)}
    assert picks == {1, 3}                                                 # 0.44 + 0.44 >= 0.5: nucleus = the two maxima
    r = Rng(8)
    picks = {sample(logits, SamplerConfig(temperature=1.0, top_p=0.3), r) for _ in range(50)}
    assert picks == {1}
    r = Rng(9)
    counts = [0] * 5
    for _ in range(4000):
        counts[sample(logits, SamplerConfig(temperature=1.0), r)] += 1
    p = torch.softmax(torch.tensor(logits), 0)
    for c, q in zip(counts, p.tolist()):
        assert abs(c / 4000 - q) < 0.03
