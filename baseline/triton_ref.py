"""Loader and runner for the reference's own Triton kernels on the GPU.

The kernels are imported, unmodified, from the copy that
``baseline/fetch_reference.py`` makes (``baseline/_ref/lazy_attn``) and compiled
by Triton for the GPU at hand when first called.  They serve two purposes and
nothing else: the GPU parity tests compare this library's output with theirs on
the same 16-bit / fp8 inputs, and ``bench.py`` times them beside this library.
The product path never imports this module.
"""
from __future__ import annotations

import sys
import types
from pathlib import Path

import torch

REF_PKG = Path(__file__).resolve().parent / "_ref" / "lazy_attn"

_loaded = None


def available() -> str:
    """'' when the reference kernels can be used here, else the reason they cannot."""
    if not (REF_PKG / "lazy" / "attention" / "ops" / "prefix_prefill.py").exists():
        return "the reference package has not been copied (baseline/fetch_reference.py)"
    if not torch.cuda.is_available():
        return "no CUDA device"
    try:
        import triton  # noqa: F401
    except Exception as e:  # pragma: no cover
        return f"triton is not importable: {e}"
    return ""


def load():
    """Import the four reference operators; returns a namespace with
    lazy_prefill, lazy_op, mepic_prefill, mepic_op."""
    global _loaded
    if _loaded is not None:
        return _loaded
    why = available()
    if why:
        raise RuntimeError(why)
    if str(REF_PKG) not in sys.path:
        sys.path.insert(0, str(REF_PKG))
    # The dispatch wrappers import a ROCm predicate from vLLM; where that module
    # does not import (other vLLM version, no ROCm libraries) a stand-in answering
    # "no" keeps the wrappers on their Triton path, which is the path under test.
    try:
        from vllm.platforms.rocm import use_rocm_custom_paged_attention  # noqa: F401
    except Exception:
        stub = types.ModuleType("vllm.platforms.rocm")
        stub.use_rocm_custom_paged_attention = lambda *a, **k: False
        sys.modules["vllm.platforms.rocm"] = stub
    from lazy.attention.ops.prefix_prefill import context_attention_fwd as lazy_prefill
    from lazy.attention.ops.chunked_prefill_paged_decode import chunked_prefill_paged_decode as lazy_op
    from lazy.attention.old_ops.prefix_prefill import context_attention_fwd as mepic_prefill
    from lazy.attention.old_ops.chunked_prefill_paged_decode import chunked_prefill_paged_decode as mepic_op
    _loaded = types.SimpleNamespace(lazy_prefill=lazy_prefill, lazy_op=lazy_op,
                                    mepic_prefill=mepic_prefill, mepic_op=mepic_op)
    return _loaded


def run(case: dict, op: str, out=None, is_mepic=True):
    """Call one reference operator on a CUDA case (the dictionaries
    ``lazy_attention_b200.synth`` builds); returns the output tensor."""
    ref = load()
    g = case["geom"]
    if out is None:
        out = torch.zeros(case["num_tokens"], g.num_q_heads, g.head_dim, dtype=case["q"].dtype,
                          device=case["q"].device)
    ks, vs = case["k_scale"].reshape(-1)[0], case["v_scale"].reshape(-1)[0]
    if op == "lazy_prefill":
        ref.lazy_prefill(case["q"], case["k"], case["v"], out, case["kv_cache_dtype"],
                         case["k_cache"], case["v_cache"], case["block_table"],
                         case["query_start_loc"], case["seq_lens"], case["max_seq_len"],
                         case["max_query_len"], ks, vs, sm_scale=case["sm_scale"],
                         cos_sin_cache=case["cos_sin_cache"], rotary_dim=g.head_dim,
                         is_lazy=case["is_lazy"], q_offset=case["q_offset"], q_mask=case["q_mask"])
    elif op == "lazy_op":
        ref.lazy_op(query=case["q"], key=case["k"], value=case["v"], output=out,
                    kv_cache_dtype=case["kv_cache_dtype"], key_cache=case["k_cache"],
                    value_cache=case["v_cache"], block_table=case["block_table"],
                    query_start_loc=case["query_start_loc"], seq_lens=case["seq_lens"],
                    max_seq_len=case["max_seq_len"], max_query_len=case["max_query_len"],
                    k_scale=ks, v_scale=vs, sm_scale=case["sm_scale"], rotary_dim=g.head_dim,
                    cos_sin_cache=case["cos_sin_cache"], is_lazy=case["is_lazy"], lazy_variant=None,
                    q_offset=case["q_offset"], q_mask=case["q_mask"],
                    packed_block_table=case["packed_block_table"])
    elif op == "mepic_prefill":
        ref.mepic_prefill(case["q"], case["k"], case["v"], out, case["kv_cache_dtype"],
                          case["k_cache"], case["v_cache"], case["block_table"],
                          case["query_start_loc"], case["seq_lens"], case["max_seq_len"],
                          case["max_query_len"], ks, vs, sm_scale=case["sm_scale"],
                          cos_sin_cache=case["cos_sin_cache"], rotary_dim=g.head_dim,
                          q_mask=case["q_mask"], q_offset=case["q_offset"], is_mepic=is_mepic)
    elif op == "mepic_op":
        ref.mepic_op(query=case["q"], key=case["k"], value=case["v"], output=out,
                     kv_cache_dtype=case["kv_cache_dtype"], key_cache=case["k_cache"],
                     value_cache=case["v_cache"], block_table=case["block_table"],
                     query_start_loc=case["query_start_loc"], seq_lens=case["seq_lens"],
                     max_seq_len=case["max_seq_len"], max_query_len=case["max_query_len"],
                     k_scale=ks, v_scale=vs, sm_scale=case["sm_scale"], rotary_dim=g.head_dim,
                     cos_sin_cache=case["cos_sin_cache"], q_offset=case["q_offset"],
                     q_mask=case["q_mask"], is_mepic=is_mepic)
    else:
        raise KeyError(op)
    return out
