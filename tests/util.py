"""Shared helpers of the test-suite: fixture loading, oracle and CUDA runners."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from lazy_attention_b200 import synth
from oracle import lazy_oracle as oracle
from oracle.runner import new_out, pack_host, run_oracle, run_oracle_by_kv_head, to_cpu_f32  # noqa: F401

GOLDEN = Path(__file__).resolve().parent / "golden"

TENSOR_KEYS = ["q", "k", "v", "k_cache", "v_cache", "block_table", "q_offset", "q_mask",
               "is_lazy", "query_start_loc", "seq_lens", "k_scale", "v_scale", "cos_sin_cache",
               "packed_block_table"]


def load_golden(name: str) -> dict:
    z = np.load(GOLDEN / f"{name}.npz")
    case = {}
    for k in TENSOR_KEYS:
        if k in z.files:
            t = torch.from_numpy(z[k])
            if k == "is_lazy":
                t = t.to(torch.bool)
            case[k] = t
    hq, hkv, d, bs, max_seq, max_q, T = (int(v) for v in z["meta"])
    case["geom"] = synth.Geometry(hq, hkv, d, bs)
    case["max_seq_len"], case["max_query_len"], case["num_tokens"] = max_seq, max_q, T
    case["sm_scale"] = float(z["sm_scale"])
    case["out"] = torch.from_numpy(z["out"])
    case["kv_cache_dtype"] = "fp8_e4m3" if case["k_cache"].dtype == torch.uint8 else "auto"
    case["sliding_window"] = int(z["sliding_window"]) if "sliding_window" in z.files else None
    case["alibi_slopes"] = torch.from_numpy(z["alibi_slopes"]) if "alibi_slopes" in z.files else None
    if "packed_block_table" not in case:
        case["packed_block_table"] = pack_host(case)
    return case


def metadata_vectors():
    return json.loads((GOLDEN / "metadata_vectors.json").read_text())


def to_device(case: dict, device) -> dict:
    return {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in case.items()}


def run_cuda(case, op: str, kernel="auto", **kw):
    """Run the library on a CUDA copy of the case; returns the output on CPU (float32)."""
    import lazy_attention_b200 as la
    c = case if case["q"].is_cuda else to_device(case, "cuda")
    out = new_out(c)
    common = dict(kv_cache_dtype=c["kv_cache_dtype"], max_seq_len=c["max_seq_len"],
                  k_scale=c["k_scale"], v_scale=c["v_scale"], sm_scale=c["sm_scale"],
                  cos_sin_cache=c["cos_sin_cache"], rotary_dim=c["geom"].head_dim,
                  sliding_window=c.get("sliding_window"), kernel=kernel)
    if kw.get("peer_out") is not None:
        common["peer_out"] = kw["peer_out"]
    if op == "lazy_prefill":
        la.context_attention_fwd(c["q"], c["k"], c["v"], out, k_cache=c["k_cache"],
                                 v_cache=c["v_cache"], b_loc=c["block_table"],
                                 b_start_loc=c["query_start_loc"], b_seq_len=c["seq_lens"],
                                 max_input_len=c["max_query_len"], is_lazy=c["is_lazy"],
                                 q_offset=c["q_offset"], q_mask=c["q_mask"],
                                 skip_decode=kw.get("skip_decode", False), **common)
    elif op == "mepic_prefill":
        la.context_attention_fwd_mepic(c["q"], c["k"], c["v"], out, k_cache=c["k_cache"],
                                       v_cache=c["v_cache"], b_loc=c["block_table"],
                                       b_start_loc=c["query_start_loc"], b_seq_len=c["seq_lens"],
                                       max_input_len=c["max_query_len"], q_offset=c["q_offset"],
                                       q_mask=c["q_mask"], is_mepic=kw.get("is_mepic", True),
                                       skip_decode=kw.get("skip_decode", False), **common)
    elif op == "lazy_op":
        la.chunked_prefill_paged_decode(
            c["q"], c["k"], c["v"], out, key_cache=c["k_cache"], value_cache=c["v_cache"],
            block_table=c["block_table"], query_start_loc=c["query_start_loc"],
            seq_lens=c["seq_lens"], max_query_len=c["max_query_len"], is_lazy=c["is_lazy"],
            q_offset=c["q_offset"], q_mask=c["q_mask"],
            packed_block_table=c["packed_block_table"], alibi_slopes=c.get("alibi_slopes"),
            **common)
    elif op == "mepic_op":
        la.chunked_prefill_paged_decode_mepic(
            c["q"], c["k"], c["v"], out, key_cache=c["k_cache"], value_cache=c["v_cache"],
            block_table=c["block_table"], query_start_loc=c["query_start_loc"],
            seq_lens=c["seq_lens"], max_query_len=c["max_query_len"], q_offset=c["q_offset"],
            q_mask=c["q_mask"], is_mepic=kw.get("is_mepic", True),
            alibi_slopes=c.get("alibi_slopes"), **common)
    else:
        raise KeyError(op)
    torch.cuda.synchronize()
    status = la.device_status()
    assert status == 0, f"a kernel reported an expired wait (code {status})"
    return out.float().cpu()


def assert_close(got, want, atol, rtol, what=""):
    diff = (got - want).abs()
    bound = atol + rtol * want.abs()
    bad = diff > bound
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} of {bad.numel()} elements off; max abs diff "
        f"{float(diff.max()):.3e} (atol {atol}, rtol {rtol})")
    assert bool(torch.isfinite(got).all()), f"{what}: non-finite output"


def slice_case(case: dict, request: int, kv_head: int) -> dict:
    """One (request, KV head) of a case as a small stand-alone case on the CPU:
    the request's pages are gathered into a compact cache (physical ids 0..n-1),
    so that the oracle can check a full-size workload one slice at a time."""
    g = case["geom"]
    G = g.num_q_heads // g.num_kv_heads
    BS = g.block_size
    qsl = case["query_start_loc"].cpu()
    s0, s1 = int(qsl[request]), int(qsl[request + 1])
    seq_len = int(case["seq_lens"][request])
    npages = (seq_len + BS - 1) // BS
    blocks = case["block_table"][request, :npages].to(torch.long).to(case["k_cache"].device)
    sub = {}
    sub["q"] = case["q"][s0:s1, G * kv_head:G * (kv_head + 1)].cpu().contiguous()
    sub["k"] = case["k"][s0:s1, kv_head:kv_head + 1].cpu().contiguous()
    sub["v"] = case["v"][s0:s1, kv_head:kv_head + 1].cpu().contiguous()
    sub["k_cache"] = case["k_cache"][blocks][:, kv_head:kv_head + 1].cpu().contiguous()
    sub["v_cache"] = case["v_cache"][blocks][:, kv_head:kv_head + 1].cpu().contiguous()
    sub["block_table"] = torch.arange(npages, dtype=torch.int32)[None, :].contiguous()
    sub["q_offset"] = case["q_offset"][request:request + 1, :npages].cpu().contiguous()
    sub["q_mask"] = case["q_mask"][request:request + 1, :npages].cpu().contiguous()
    sub["is_lazy"] = case["is_lazy"][request:request + 1].cpu()
    sub["query_start_loc"] = torch.tensor([0, s1 - s0], dtype=torch.int32)
    sub["seq_lens"] = torch.tensor([seq_len], dtype=torch.int32)
    for k in ("k_scale", "v_scale", "cos_sin_cache"):
        sub[k] = case[k].cpu()
    sub["geom"] = synth.Geometry(G, 1, g.head_dim, BS)
    sub["num_tokens"] = s1 - s0
    sub["max_query_len"] = s1 - s0
    sub["max_seq_len"] = seq_len
    sub["sm_scale"] = case["sm_scale"]
    sub["kv_cache_dtype"] = case["kv_cache_dtype"]
    sub["sliding_window"] = case.get("sliding_window")
    sub["packed_block_table"] = pack_host(sub)
    sub["token_range"] = (s0, s1)
    sub["head_range"] = (G * kv_head, G * (kv_head + 1))
    return sub
