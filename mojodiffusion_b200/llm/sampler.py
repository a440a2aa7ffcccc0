"""Host-side next-token sampler: greedy, temperature, top-k, top-p (nucleus), driven by an xorshift64* generator whose
uniform is the top 53 bits of the 64-bit output over 2^53, so it spans the whole of [0, 1). Candidates are ordered by
descending logit (ties keep vocabulary order), top-k restricts the candidate set before the temperature softmax, top-p
keeps the shortest prefix whose cumulative probability reaches p and renormalises over it
(serenitymojo/llm/sampler.mojo:15-141)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

_M64 = (1 << 64) - 1


class Rng:
    def __init__(self, seed: int):
        s = seed & _M64
        self.state = s if s != 0 else 0x9E3779B97F4A7C15       # zero is the fixed point of xorshift

    def next_u64(self) -> int:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & _M64
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & _M64

    def next_f64(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / 9007199254740992.0)


@dataclass
class SamplerConfig:
    temperature: float = 1.0     # <= 0: greedy
    top_k: int = 0               # <= 0: off
    top_p: float = 1.0           # outside (0, 1): off
    seed: int = 0


def argmax(logits: Sequence[float]) -> int:
    best, bestv = 0, logits[0]
    for i in range(1, len(logits)):
        if logits[i] > bestv:
            best, bestv = i, logits[i]
    return best


def sample(logits: Sequence[float], cfg: SamplerConfig, rng: Rng) -> int:
    n = len(logits)
    if n == 0:
        raise ValueError("sample: empty logits")
    if cfg.temperature <= 0.0:
        return argmax(logits)
    order = sorted(range(n), key=lambda i: -float(logits[i]))            # stable: ties keep vocabulary order
    keep = cfg.top_k if 0 < cfg.top_k < n else n
    inv_t = 1.0 / cfg.temperature
    maxl = float(logits[order[0]]) * inv_t
    probs = [math.exp(float(logits[order[i]]) * inv_t - maxl) for i in range(keep)]
    total = sum(probs)
    probs = [p / total for p in probs]
    cutoff = keep
    if 0.0 < cfg.top_p < 1.0:
        cum, cutoff = 0.0, 0
        for i in range(keep):
            cum += probs[i]
            cutoff = i + 1
            if cum >= cfg.top_p:
                break
        renorm = sum(probs[:cutoff])
        probs = [p / renorm for p in probs[:cutoff]]
    u = rng.next_f64()
    acc = 0.0
    for i in range(cutoff):
        acc += probs[i]
        if u < acc:
            return order[i]
    return order[cutoff - 1]
