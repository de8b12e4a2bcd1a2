"""Prefix-prefill for callers that cannot allocate device memory.

``context_attention_fwd`` hands the split-KV kernel a scratch tensor that this
package allocates with torch.  An engine that has given all free HBM to the KV
cache, or that calls the layer where ``cudaMalloc`` and its implicit device
synchronisation are not allowed, cannot do that.  :func:`context_attention_fwd_no_alloc`
takes the same tensors and calls ``la_prefill_fwd_noalloc`` instead, which keeps
the partial results in a 32 MiB array inside the library; no tensor is created
and no allocator is called on the way.

Limits: bf16/fp16 activations and cache, head size 64 or 128, page size 16, no
sliding window (what the tensor-core kernel takes), and a call whose scratch need
(``la_prefill_workspace_bytes``) is at most 32 MiB -- larger calls are refused
with an error that states both sizes.  All calls on one GPU share the array, so
calls that overlap on the GPU (different streams) race; make the first call on
a device outside any stream capture.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_ACT = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16}

#: Size of the scratch array inside the library (bytes).
NO_ALLOC_SCRATCH_BYTES = 32 << 20


def scratch_need(*args, **kwargs) -> int:
    """Bytes of split-KV scratch the call described by the arguments of
    :func:`context_attention_fwd_no_alloc` needs (0 when it does not split)."""
    a = _build_args(*args, **kwargs)
    return int(_lib.load().la_prefill_workspace_bytes(C.byref(a)))


def context_attention_fwd_no_alloc(*args, **kwargs) -> None:
    """Same result as ``context_attention_fwd`` (or its per-token twin when
    ``rot_mode`` is ``ROT_MEPIC``), written into ``o``; allocates nothing.

    Arguments: ``q, k, v, o, k_cache, v_cache, b_loc, b_start_loc, b_seq_len,
    max_seq_len, max_input_len`` and the keywords ``cos_sin_cache, is_lazy,
    q_offset, q_mask, sm_scale, skip_decode, rot_mode, is_mepic``."""
    a = _build_args(*args, **kwargs)
    q = args[0]
    lib = _lib.load()
    with torch.cuda.device(q.device):
        rc = lib.la_prefill_fwd_noalloc(C.byref(a), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(rc, "la_prefill_fwd_noalloc")


def _build_args(q, k, v, o, k_cache, v_cache, b_loc, b_start_loc, b_seq_len,
                max_seq_len, max_input_len, cos_sin_cache=None, is_lazy=None,
                q_offset=None, q_mask=None, sm_scale=None, skip_decode=False,
                rot_mode: int = _lib.ROT_LAZY, is_mepic: bool = False, packed_block_table=None):
    """Same checks and struct filling as the regular operators (one shared helper), for
    16-bit caches; creates no tensor."""
    if q.dtype not in _ACT or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("q, k, v, o and the caches must share one dtype out of float16/bfloat16")
    from .attention import prefill_args
    return prefill_args(q, k, v, o, "auto", k_cache, v_cache, b_loc, b_start_loc, b_seq_len,
                        max_seq_len, max_input_len, None, None, None, None, sm_scale, skip_decode,
                        cos_sin_cache, None, True, is_lazy, q_offset, q_mask, int(rot_mode),
                        bool(is_mepic), "tensor", None, packed_block_table)
