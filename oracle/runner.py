"""Runs the CPU oracle on a case dictionary.  TEST INFRASTRUCTURE ONLY.

The case dictionaries are the ones ``lazy_attention_b200.synth`` builds and the
golden fixtures load into.  Used by ``tests/``, by ``__graft_entry__.smoke`` and
by the CPU-baseline / reference legs of ``bench.py``; never by the product path.
"""
from __future__ import annotations

import torch

from . import lazy_oracle as oracle


def pack_host(case):
    return torch.from_numpy(oracle.pack_block_table(case["block_table"].cpu().numpy(),
                                                    case["q_offset"].cpu().numpy(),
                                                    case["q_mask"].cpu().numpy()))


def to_cpu_f32(case: dict) -> dict:
    """CPU copy of a case with float tensors widened to float32 (the oracle's input)."""
    out = {}
    for k, v in case.items():
        if torch.is_tensor(v):
            v = v.detach().cpu()
            if v.dtype in (torch.float16, torch.bfloat16):
                v = v.to(torch.float32)
        out[k] = v
    return out


def new_out(case, device=None, dtype=None):
    q = case["q"]
    return torch.zeros(case["num_tokens"], q.shape[1], q.shape[2], dtype=dtype or q.dtype,
                       device=device or q.device)


def run_oracle(case, op: str, **kw):
    """op: lazy_prefill | lazy_op | mepic_op | mepic_prefill.  Returns float32 output."""
    c = to_cpu_f32(case)
    out = new_out(c, dtype=torch.float32)
    ks, vs = c["k_scale"].reshape(-1)[0], c["v_scale"].reshape(-1)[0]
    common = dict(kv_cache_dtype=c["kv_cache_dtype"], max_seq_len=c["max_seq_len"],
                  k_scale=ks, v_scale=vs, sm_scale=c["sm_scale"], cos_sin_cache=c["cos_sin_cache"],
                  rotary_dim=c["geom"].head_dim, sliding_window=c.get("sliding_window"))
    if op == "lazy_prefill":
        oracle.context_attention_fwd(c["q"], c["k"], c["v"], out, k_cache=c["k_cache"],
                                     v_cache=c["v_cache"], b_loc=c["block_table"],
                                     b_start_loc=c["query_start_loc"], b_seq_len=c["seq_lens"],
                                     max_input_len=c["max_query_len"], is_lazy=c["is_lazy"],
                                     q_offset=c["q_offset"], q_mask=c["q_mask"],
                                     skip_decode=kw.get("skip_decode", False), **common)
    elif op == "mepic_prefill":
        oracle.context_attention_fwd_mepic(c["q"], c["k"], c["v"], out, k_cache=c["k_cache"],
                                           v_cache=c["v_cache"], b_loc=c["block_table"],
                                           b_start_loc=c["query_start_loc"],
                                           b_seq_len=c["seq_lens"],
                                           max_input_len=c["max_query_len"],
                                           q_offset=c["q_offset"], q_mask=c["q_mask"],
                                           is_mepic=kw.get("is_mepic", True),
                                           skip_decode=kw.get("skip_decode", False), **common)
    elif op == "lazy_op":
        oracle.chunked_prefill_paged_decode(
            c["q"], c["k"], c["v"], out, key_cache=c["k_cache"], value_cache=c["v_cache"],
            block_table=c["block_table"], query_start_loc=c["query_start_loc"],
            seq_lens=c["seq_lens"], max_query_len=c["max_query_len"], is_lazy=c["is_lazy"],
            q_offset=c["q_offset"], q_mask=c["q_mask"],
            packed_block_table=c["packed_block_table"], alibi_slopes=c.get("alibi_slopes"),
            round_q_to=kw.get("round_q_to"), **common)
    elif op == "mepic_op":
        oracle.chunked_prefill_paged_decode_mepic(
            c["q"], c["k"], c["v"], out, key_cache=c["k_cache"], value_cache=c["v_cache"],
            block_table=c["block_table"], query_start_loc=c["query_start_loc"],
            seq_lens=c["seq_lens"], max_query_len=c["max_query_len"], q_offset=c["q_offset"],
            q_mask=c["q_mask"], is_mepic=kw.get("is_mepic", True),
            alibi_slopes=c.get("alibi_slopes"), **common)
    else:
        raise KeyError(op)
    return out



def kv_head_slice(case: dict, kv_head: int) -> dict:
    """The call restricted to one KV head and its query heads (views, no copies):
    attention is independent per KV head, so running the slices one after the other
    is the same computation as the whole call with a fraction of the memory."""
    g = case["geom"]
    G = g.num_q_heads // g.num_kv_heads
    sub = dict(case)
    sub["q"] = case["q"][:, G * kv_head:G * (kv_head + 1)]
    sub["k"] = case["k"][:, kv_head:kv_head + 1]
    sub["v"] = case["v"][:, kv_head:kv_head + 1]
    sub["k_cache"] = case["k_cache"][:, kv_head:kv_head + 1]
    sub["v_cache"] = case["v_cache"][:, kv_head:kv_head + 1]
    sub["geom"] = type(g)(G, 1, g.head_dim, g.block_size, g.rope_theta)
    if case.get("alibi_slopes") is not None:
        sub["alibi_slopes"] = case["alibi_slopes"][G * kv_head:G * (kv_head + 1)]
    return sub


def run_oracle_by_kv_head(case, op: str, **kw):
    """run_oracle one KV head at a time (bounded memory for long contexts)."""
    g = case["geom"]
    G = g.num_q_heads // g.num_kv_heads
    out = new_out(case, device="cpu", dtype=torch.float32)
    for h in range(g.num_kv_heads):
        out[:, G * h:G * (h + 1)] = run_oracle(kv_head_slice(case, h), op, **kw)
    return out
