"""Prompt-expansion language model support: KV-cached incremental decode over the Qwen3 stack (:mod:`decoder`) and the
host-side token sampler (:mod:`sampler`)."""
from .decoder import KVCache, Qwen3Decoder, single_query_attention
from .sampler import Rng, SamplerConfig, argmax, sample

__all__ = ["KVCache", "Qwen3Decoder", "single_query_attention", "Rng", "SamplerConfig", "argmax", "sample"]
