"""Row plan of variable-length guidance with a key / value cache for the Lance text-to-video model (metadata only).

A Lance sequence is [text prefix, visual-start token, generated latent tokens, visual-end token]. With a cache the
conditional branch prefills the text prefix once (causally) and every denoise step only queries the visual rows; the
text-unconditional branch DROPS the text prefix instead of padding it, so its rows are the same visual rows shifted down
by the prefix length and its cache is empty. The records below say, per branch and layer, which source rows are queried,
where they sit in the packed (shortened) sequence, how long the attention key range is and how much the prefill writes.
Behaviour: serenitymojo/models/lance/cfg_kv_cache.mojo:11-295.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

BRANCH_COND, BRANCH_TEXT_UNCOND = 0, 1


@dataclass(frozen=True)
class LanceInput:
    full_ids: Sequence[int]
    t_pos: Sequence[int]
    h_pos: Sequence[int]
    w_pos: Sequence[int]
    text_split_len: int
    gen_start: int
    gen_len: int
    latent_pos_ids: Sequence[int]


@dataclass(frozen=True)
class KVBranchPlan:
    prefix_len: int
    query_start: int
    query_len: int
    query_gen_start: int
    query_gen_len: int
    packed_index_shift: int
    prefill_updates_cache: bool
    prefill_is_causal: bool

    @property
    def query_end(self) -> int:
        return self.query_start + self.query_len

    def kv_elements_per_layer(self, kv_heads: int, head_dim: int) -> int:
        return self.prefix_len * kv_heads * head_dim * 2          # K and V, cached after rotary, before head repetition


@dataclass(frozen=True)
class KVLayerCall:
    branch_id: int
    layer_idx: int
    source_query_start: int
    query_len: int
    packed_query_start: int
    local_gen_start: int
    gen_len: int
    prefix_cache_len: int
    query_kv_start: int
    attention_kv_len: int
    prefix_cache_write_len: int
    prefix_cache_is_causal: bool

    @property
    def packed_query_end(self) -> int:
        return self.packed_query_start + self.query_len

    @property
    def local_gen_end(self) -> int:
        return self.local_gen_start + self.gen_len


@dataclass(frozen=True)
class CfgKVPlan:
    cond: KVBranchPlan
    text_uncond: KVBranchPlan
    dropped_text_len: int
    gen_len: int
    cond_total_len: int
    uncond_query_len: int

    def total_kv_bytes(self, layers: int, kv_heads: int, head_dim: int, dtype_bytes: int = 2) -> int:
        per = self.cond.kv_elements_per_layer(kv_heads, head_dim) + self.text_uncond.kv_elements_per_layer(kv_heads, head_dim)
        return per * dtype_bytes * layers


def validate_input(inp: LanceInput, name: str = "cond") -> None:
    total = len(inp.full_ids)
    if not (total == len(inp.t_pos) == len(inp.h_pos) == len(inp.w_pos)):
        raise ValueError(f"{name}: token ids and position ids must have equal length")
    if inp.text_split_len <= 0 or inp.gen_len <= 0:
        raise ValueError(f"{name}: text_split_len and gen_len must be positive")
    if inp.gen_start != inp.text_split_len + 1:
        raise ValueError(f"{name}: gen_start must point after the visual start token")
    if total != inp.text_split_len + 1 + inp.gen_len + 1:
        raise ValueError(f"{name}: expected [text prefix, visual start, gen tokens, visual end]")
    if len(inp.latent_pos_ids) != inp.gen_len:
        raise ValueError(f"{name}: latent_pos_ids length must equal gen_len")


def text_drop_plan(cond: LanceInput) -> CfgKVPlan:
    validate_input(cond)
    q = cond.gen_len + 2
    return CfgKVPlan(KVBranchPlan(cond.text_split_len, cond.text_split_len, q, 1, cond.gen_len, 0, True, True),
                     KVBranchPlan(0, cond.text_split_len, q, 1, cond.gen_len, cond.text_split_len, False, False),
                     cond.text_split_len, cond.gen_len, len(cond.full_ids), q)


def layer_call(plan: CfgKVPlan, branch_id: int, layer_idx: int) -> KVLayerCall:
    if branch_id not in (BRANCH_COND, BRANCH_TEXT_UNCOND):
        raise ValueError(f"invalid branch id {branch_id}")
    b = plan.cond if branch_id == BRANCH_COND else plan.text_uncond
    if layer_idx < 0 or b.prefix_len < 0 or b.query_start < 0 or b.query_len <= 0 or b.packed_index_shift < 0:
        raise ValueError("layer call: negative index or empty query span")
    if b.query_start < b.packed_index_shift or b.query_gen_start < 0 or b.query_gen_len < 0:
        raise ValueError("layer call: packed query start or generated span out of range")
    if b.query_gen_start + b.query_gen_len > b.query_len:
        raise ValueError("layer call: generated span exceeds query span")
    return KVLayerCall(branch_id, layer_idx, b.query_start, b.query_len, b.query_start - b.packed_index_shift, b.query_gen_start,
                       b.query_gen_len, b.prefix_len, b.prefix_len, b.prefix_len + b.query_len,
                       b.prefix_len if b.prefill_updates_cache else 0, b.prefill_is_causal)


def validate_plan(inp: LanceInput, plan: CfgKVPlan, layers: int, latent_thw: Sequence[int]) -> None:
    """Every consistency rule between an input, its plan and the latent grid; raises ValueError naming the first violation."""
    validate_input(inp)
    t, h, w = latent_thw
    if min(t, h, w) <= 0 or layers <= 0:
        raise ValueError("latent dimensions and depth must be positive")
    gen = t * h * w
    checks = [
        (inp.gen_len == gen and plan.gen_len == gen, "gen_len does not match latent dimensions"),
        (plan.cond_total_len == len(inp.full_ids), "cond_total_len does not match input length"),
        (plan.dropped_text_len == inp.text_split_len, "dropped text length must equal text prefix"),
        (plan.cond.prefix_len == inp.text_split_len and plan.cond.query_start == inp.text_split_len, "cond prefix / query start"),
        (plan.cond.query_len == gen + 2 and plan.cond.query_end == len(inp.full_ids), "cond query must cover visual start / gen / end"),
        (plan.cond.packed_index_shift == 0, "cond packed shift must be zero"),
        (plan.text_uncond.query_len == plan.cond.query_len == plan.uncond_query_len, "uncond query length must match cond"),
        (plan.text_uncond.prefix_len == 0, "uncond prefix cache must be empty"),
        (plan.text_uncond.query_start == plan.cond.query_start, "uncond source query must match cond query"),
        (plan.text_uncond.packed_index_shift == inp.text_split_len, "uncond packed shift must drop text prefix"),
    ]
    c, u = layer_call(plan, BRANCH_COND, layers - 1), layer_call(plan, BRANCH_TEXT_UNCOND, layers - 1)
    checks += [
        (c.attention_kv_len == len(inp.full_ids), "cond attention length must equal the full sequence"),
        (u.attention_kv_len == plan.uncond_query_len, "uncond attention length must equal the query sequence"),
        (c.query_kv_start == inp.text_split_len and u.query_kv_start == 0, "query K / V placement"),
        (c.packed_query_end == len(inp.full_ids) and u.packed_query_end == plan.uncond_query_len, "packed query end"),
        (c.local_gen_start == u.local_gen_start == 1 and c.local_gen_end == u.local_gen_end == gen + 1, "generated span must skip start / end tokens"),
        (c.prefix_cache_write_len == inp.text_split_len and u.prefix_cache_write_len == 0, "prefill write lengths"),
    ]
    for ok, msg in checks:
        if not ok:
            raise ValueError("Lance CFG KV plan: " + msg)
