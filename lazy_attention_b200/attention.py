"""Host-side mirror of the reference's attention operators.

The four functions keep the reference's names, argument order, argument
meaning and error behaviour, and forward to the C ABI
(``include/lazy_attention_b200.h``):

* :func:`context_attention_fwd`  -- lazy_attn/lazy/attention/ops/prefix_prefill.py:600-744
* :func:`chunked_prefill_paged_decode` -- lazy_attn/lazy/attention/ops/chunked_prefill_paged_decode.py:36-221
* :func:`context_attention_fwd_mepic` -- lazy_attn/lazy/attention/old_ops/prefix_prefill.py:411-555
* :func:`chunked_prefill_paged_decode_mepic` -- lazy_attn/lazy/attention/old_ops/chunked_prefill_paged_decode.py:283-442

Differences by design: no device->host sync (the reference's ``.item()`` at
ops/chunked_prefill_paged_decode.py:156 is gone), no per-call tensor
allocation except the cached split-KV scratch, and the work runs on the current
CUDA stream of the tensors' device.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _lib
from ._lib import LaDecodeArgs, LaPrefillArgs

_ACT = {torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16,
        torch.bfloat16: _lib.DTYPE_BF16}

_workspaces = {}
_retired_workspaces = []  # outgrown buffers stay allocated: captured CUDA graphs may still point at them


def device_status() -> int:
    """Synchronise and return (then clear) the status word that kernels with
    bounded waits set when a wait expires; 0 means none did."""
    return int(_lib.load().la_device_status())


def check_device() -> None:
    """Synchronise and raise ``RuntimeError`` if a kernel of this library gave up on a
    bounded wait since the last check (its results are then invalid).  The operators do
    not synchronise, so they cannot report this themselves: an engine that uses the
    patch-in calls this once per step, or every few steps."""
    _lib.check(_lib.load().la_check_device(), "la_check_device")


def launch_count() -> int:
    """Kernels launched by the library in this process."""
    return int(_lib.load().la_launch_count())


def _workspace(device: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Scratch for the split-KV kernels, owned by this module, grown on demand: one buffer per
    device and stream, so that calls on different streams never share partial results."""
    if nbytes <= 0:
        return None
    if torch.cuda.is_current_stream_capturing():
        # like any temporary of a captured region: it lives in the graph's memory pool, stays
        # reserved for the graph's replays and goes with the graph
        return torch.empty(int(nbytes) + 256, dtype=torch.uint8, device=device)
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def reserve_workspace(device, nbytes: int) -> None:
    """Grow the split-KV scratch of this device's current stream to at least ``nbytes`` now, so
    that later calls do not allocate.  Calls on one stream share it (they are ordered); every
    other stream gets a buffer of its own; a call made under stream capture takes a temporary
    from the graph's memory pool instead."""
    _workspace(torch.device(device), int(nbytes))


def _env_flag(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() in ("1", "true", "yes", "on")


def _kernel_choice(kernel) -> int:
    if kernel is None:
        kernel = os.environ.get("LAZY_ATTN_B200_KERNEL", "auto")
    if isinstance(kernel, int):
        return kernel
    return {"auto": _lib.KERNEL_AUTO, "general": _lib.KERNEL_GENERAL,
            "tensor": _lib.KERNEL_TENSOR}[str(kernel).lower()]


def _fp8_view(kv_cache_dtype: str, k_cache, v_cache):
    """Cache dtype resolution, as the reference wrappers do it
    (ops/prefix_prefill.py:637-654)."""
    kv_code = None
    if "fp8" in kv_cache_dtype:
        assert k_cache.dtype == torch.uint8
        assert v_cache.dtype == torch.uint8
        if kv_cache_dtype in ("fp8", "fp8_e4m3"):
            kv_code = _lib.DTYPE_FP8_E4M3
        elif kv_cache_dtype == "fp8_e5m2":
            kv_code = _lib.DTYPE_FP8_E5M2
        else:
            raise ValueError("Unsupported FP8 dtype:", kv_cache_dtype)
    elif k_cache.dtype == torch.float8_e4m3fn:
        kv_code = _lib.DTYPE_FP8_E4M3
    elif k_cache.dtype == torch.float8_e5m2:
        kv_code = _lib.DTYPE_FP8_E5M2
    if kv_code is None and (k_cache.dtype == torch.uint8 or
                            (v_cache.dtype == torch.uint8 and kv_cache_dtype == "auto")):
        raise ValueError("kv_cache_dtype='auto' unsupported for FP8 KV Cache prefill kernel")
    if kv_code is None:
        if k_cache.dtype not in _ACT:
            raise ValueError(f"unsupported cache dtype {k_cache.dtype}")
        kv_code = _ACT[k_cache.dtype]
    return kv_code


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("lazy_attention_b200 runs on CUDA tensors only (no CPU path)")


def _cache_strides(k_cache, v_cache):
    # K [nb, Hkv, D/x, BS, x], V [nb, Hkv, D, BS]; the page of one head is dense.
    nb, hkv, dx, bs, x = k_cache.shape
    if k_cache.stride(4) != 1 or k_cache.stride(3) != x or k_cache.stride(2) != bs * x:
        raise ValueError("k_cache: the [D/x, BS, x] page of a head must be contiguous")
    if v_cache.stride(3) != 1 or v_cache.stride(2) != v_cache.shape[3]:
        raise ValueError("v_cache: the [D, BS] page of a head must be contiguous")
    return bs, x


def _ptr(t):
    return None if t is None else t.data_ptr()


def _i32(t, name):
    if t is not None and t.dtype != torch.int32:
        raise ValueError(f"{name} must be int32")
    return t


def _bool_u8(t):
    if t is None:
        return None
    if t.dtype == torch.bool:
        return t.view(torch.uint8)
    if t.dtype == torch.uint8:
        return t
    raise ValueError("is_lazy must be a bool tensor")


def _slots(slot_mapping, num_rows):
    """Pointer of the slot mapping of a fused cache write (None: off)."""
    if slot_mapping is None:
        return None
    if slot_mapping.dtype != torch.int64 or not slot_mapping.is_cuda or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 CUDA tensor")
    return slot_mapping.data_ptr()


def _positions(positions):
    """Pointer of the token positions of a fused rotary op (None: the query is already rotated)."""
    if positions is None:
        return None
    if positions.dtype != torch.int64 or not positions.is_cuda or not positions.is_contiguous():
        raise ValueError("positions must be a contiguous int64 CUDA tensor")
    return positions.data_ptr()


def _scale(t, device):
    if torch.is_tensor(t):
        if t.dtype != torch.float32 or not t.is_cuda:
            raise ValueError("k_scale / v_scale must be float32 CUDA tensors")
        return t
    raise ValueError("k_scale / v_scale must be 1-element float32 device tensors")


def prefill_args(q, k, v, o, kv_cache_dtype, k_cache, v_cache, b_loc, b_start_loc, b_seq_len,
                 max_seq_len, max_input_len, k_scale, v_scale, alibi_slopes, sliding_window,
                 sm_scale, skip_decode, cos_sin_cache, rotary_dim, is_neox_style, is_lazy,
                 q_offset, q_mask, rot_mode, is_mepic, kernel, peer_out=None,
                 packed_block_table=None, slot_mapping=None, positions=None) -> LaPrefillArgs:
    """Checks the tensors of a prefix-prefill call the way the reference wrapper does
    (ops/prefix_prefill.py:626-674: fp8 views, dtype and shape assertions, alibi refusal)
    plus what a raw-pointer interface must know (devices, dtypes of the int tables, unit
    inner strides, page contiguity), and fills the C struct.  Every entry point that takes
    ``LaPrefillArgs`` goes through here.  The workspace fields are left empty."""
    kv_code = _fp8_view(kv_cache_dtype, k_cache, v_cache)
    Lq, Lk, Lv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Lq == Lk and Lk == Lv
    if sm_scale is None:
        sm_scale = 1.0 / (Lq ** 0.5)
    batch = b_seq_len.shape[0]
    assert batch + 1 == len(b_start_loc)
    if sliding_window is None or sliding_window <= 0:
        sliding_window = 0
    if alibi_slopes is not None:
        raise NotImplementedError("Alibi slopes are not implemented for prefix prefill")
    if not is_neox_style:
        raise NotImplementedError("only NeoX-style rotary embedding is supported")
    _require_cuda(q, k, v, o, k_cache, v_cache, b_loc, b_start_loc, b_seq_len, q_offset, q_mask,
                  packed_block_table, is_lazy)
    if q.dtype not in _ACT or k.dtype != q.dtype or v.dtype != q.dtype or o.dtype != q.dtype:
        raise ValueError("q, k, v, o must share one dtype out of float32/float16/bfloat16")
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (o, "o")):
        if t.stride(2) != 1:
            raise ValueError(f"{n}: last dimension must be contiguous")
    bs, x = _cache_strides(k_cache, v_cache)
    _i32(b_loc, "b_loc"); _i32(b_start_loc, "b_start_loc"); _i32(b_seq_len, "b_seq_len")
    _i32(q_offset, "q_offset"); _i32(q_mask, "q_mask")
    if b_loc.stride(1) != 1:
        raise ValueError("b_loc must have unit inner stride")
    for t, n in ((q_offset, "q_offset"), (q_mask, "q_mask")):
        if t is not None and (t.stride(0) != b_loc.stride(0) or t.stride(1) != 1):
            # the kernels index both with the block table's strides
            raise ValueError(f"{n} must share the block table's strides")
    if rotary_dim is None:
        rotary_dim = Lq
    a = LaPrefillArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.q_stride_t, a.q_stride_h = q.stride(0), q.stride(1)
    a.k_stride_t, a.k_stride_h = k.stride(0), k.stride(1)
    a.v_stride_t, a.v_stride_h = v.stride(0), v.stride(1)
    a.o_stride_t, a.o_stride_h = o.stride(0), o.stride(1)
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.kc_stride_block, a.kc_stride_head = k_cache.stride(0), k_cache.stride(1)
    a.vc_stride_block, a.vc_stride_head = v_cache.stride(0), v_cache.stride(1)
    a.num_blocks = k_cache.shape[0]
    a.block_table, a.q_offset, a.q_mask = _ptr(b_loc), _ptr(q_offset), _ptr(q_mask)
    a.table_stride = b_loc.stride(0)
    if packed_block_table is not None:
        if packed_block_table.dtype != torch.int64 or packed_block_table.stride(1) != 1:
            raise ValueError("packed_block_table must be int64 with unit inner stride")
        if packed_block_table.shape[0] < batch:
            raise ValueError("packed_block_table has fewer rows than the batch")
        a.packed_block_table = packed_block_table.data_ptr()
        a.packed_stride = packed_block_table.stride(0)
    a.slot_mapping = _slots(slot_mapping, q.shape[0])
    a.q_positions = _positions(positions)
    a.query_start_loc, a.seq_lens = b_start_loc.data_ptr(), b_seq_len.data_ptr()
    a.is_lazy = _ptr(_bool_u8(is_lazy))  # a view of the caller's tensor: same storage
    if kv_code in (_lib.DTYPE_FP8_E4M3, _lib.DTYPE_FP8_E5M2) or k_scale is not None:
        ks, vs = _scale(k_scale, q.device), _scale(v_scale, q.device)
        a.k_scale, a.v_scale = ks.data_ptr(), vs.data_ptr()
    if cos_sin_cache is not None:
        _require_cuda(cos_sin_cache)
        if cos_sin_cache.dtype not in _ACT or not cos_sin_cache.is_contiguous():
            raise ValueError("cos_sin_cache must be a contiguous f32/f16/bf16 tensor")
        if cos_sin_cache.shape[-1] != rotary_dim:
            raise ValueError("cos_sin_cache rows must hold rotary_dim values")
        a.cos_sin_cache = cos_sin_cache.data_ptr()
        a.cos_sin_rows = cos_sin_cache.shape[0]
        a.cos_sin_dtype = _ACT[cos_sin_cache.dtype]
    a.batch = batch
    a.num_q_heads, a.num_kv_heads, a.head_dim = q.shape[1], k.shape[1], Lq
    a.block_size, a.x = bs, x
    a.max_query_len = int(max_input_len)
    a.max_seq_len = int(max_seq_len) if max_seq_len else 0
    a.q_dtype, a.kv_dtype = _ACT[q.dtype], kv_code
    a.rotary_dim = int(rotary_dim)
    a.sliding_window = int(sliding_window)
    a.skip_decode = int(bool(skip_decode))
    a.rot_mode, a.is_mepic = rot_mode, int(bool(is_mepic))
    a.sm_scale = float(sm_scale)
    a.kernel = _kernel_choice(kernel)
    if peer_out is not None:
        peer_out.fill(a.peer)
    return a


def _prefill(q, k, v, o, *rest, **kw):
    a = prefill_args(q, k, v, o, *rest, **kw)
    lib = _lib.load()
    need = lib.la_prefill_workspace_bytes(C.byref(a))
    ws = _workspace(q.device, need)
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(q.device):
        rc = lib.la_prefill_fwd(C.byref(a), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(rc, "la_prefill_fwd")


@torch.inference_mode()
def context_attention_fwd(q, k, v, o, kv_cache_dtype: str, k_cache, v_cache, b_loc, b_start_loc,
                          b_seq_len, max_seq_len, max_input_len, k_scale: torch.Tensor,
                          v_scale: torch.Tensor, alibi_slopes=None, sliding_window=None,
                          sm_scale=None, skip_decode=False, cos_sin_cache=None, rotary_dim=None,
                          is_neox_style=True, is_lazy=None, q_offset=None, q_mask=None,
                          kernel=None, peer_out=None, packed_block_table=None, slot_mapping=None,
                          positions=None):
    """Prefix-prefill attention, per-page rotation variant.  Writes ``o`` in place.

    For a lazy request every cached page's K is rotated forward by
    ``q_offset - 1`` positions (0 and 1 mean none) and the last ``q_mask``
    tokens of the page are masked; the new tokens attend causally to the new
    K/V.  Requests whose ``is_lazy`` is false take the plain paged path.

    ``packed_block_table`` (not in the reference's signature; the runner keeps it
    for the decode kernel) lets the kernel read a page's block id, offset and pad
    count as one 8-byte entry instead of three gathers.  ``slot_mapping`` (also an
    addition) makes the call store the new K/V rows into the caches itself: the
    ``write_to_paged_cache`` that precedes the op in the reference backend
    (backends/triton_attn.py:100-109) is then not needed.  ``positions`` (int64 per
    token, an addition too) fuses the query-only rotary op that runs just before the
    attention op (model_executor/layers/rotary_embedding.py:66-94): ``q`` is then
    passed without rotary embedding and is rotated as the kernel stages it.
    """
    _prefill(q, k, v, o, kv_cache_dtype, k_cache, v_cache, b_loc, b_start_loc, b_seq_len,
             max_seq_len, max_input_len, k_scale, v_scale, alibi_slopes, sliding_window,
             sm_scale, skip_decode, cos_sin_cache, rotary_dim, is_neox_style, is_lazy,
             q_offset, q_mask, _lib.ROT_LAZY, False, kernel, peer_out, packed_block_table, slot_mapping,
             positions)


@torch.inference_mode()
def context_attention_fwd_mepic(q, k, v, o, kv_cache_dtype: str, k_cache, v_cache, b_loc,
                                b_start_loc, b_seq_len, max_seq_len, max_input_len,
                                k_scale: torch.Tensor, v_scale: torch.Tensor, alibi_slopes=None,
                                sliding_window=None, sm_scale=None, skip_decode=False,
                                cos_sin_cache=None, rotary_dim=None, is_neox_style=True,
                                q_mask=None, q_offset=None, is_mepic: bool = True,
                                force_fp32_rotary: bool = False, kernel=None, peer_out=None,
                                packed_block_table=None, slot_mapping=None, positions=None):
    """Prefix-prefill attention, per-token rotation variant: cached K is rotated
    at each token's slot position, new K at ``ctx_len + n``.  The tensor-core
    kernels evaluate the rotation in packed 16-bit arithmetic (the reference's
    default), the general kernel in float32; ``force_fp32_rotary`` is accepted and
    does not change the kernel -- the two evaluations differ by rounding only."""
    _prefill(q, k, v, o, kv_cache_dtype, k_cache, v_cache, b_loc, b_start_loc, b_seq_len,
             max_seq_len, max_input_len, k_scale, v_scale, alibi_slopes, sliding_window,
             sm_scale, skip_decode, cos_sin_cache, rotary_dim, is_neox_style, None,
             q_offset, q_mask, _lib.ROT_MEPIC, is_mepic, kernel, peer_out, packed_block_table, slot_mapping,
             positions)


def _decode(query, output, kv_cache_dtype, key_cache, value_cache, query_start_loc, seq_lens,
            max_seq_len, k_scale, v_scale, alibi_slopes, sliding_window, sm_scale, rotary_dim,
            cos_sin_cache, is_lazy, packed_block_table, block_table, q_mask, rot_mode,
            ignore_q_mask, kernel, peer_out=None, key=None, value=None, slot_mapping=None, positions=None,
            rope_meta=None):
    kv_code = _fp8_view(kv_cache_dtype, key_cache, value_cache)
    _require_cuda(query, output, key_cache, value_cache, query_start_loc, seq_lens)
    if query.dtype not in _ACT or output.dtype != query.dtype:
        raise ValueError("query and output must share one dtype out of float32/float16/bfloat16")
    if query.stride(2) != 1 or output.stride(2) != 1:
        raise ValueError("query / output: last dimension must be contiguous")
    bs, x = _cache_strides(key_cache, value_cache)
    _i32(query_start_loc, "query_start_loc"); _i32(seq_lens, "seq_lens")
    a = LaDecodeArgs()
    a.q, a.out = query.data_ptr(), output.data_ptr()
    a.q_stride_t, a.q_stride_h = query.stride(0), query.stride(1)
    a.o_stride_t, a.o_stride_h = output.stride(0), output.stride(1)
    a.k_cache, a.v_cache = key_cache.data_ptr(), value_cache.data_ptr()
    a.kc_stride_block, a.kc_stride_head = key_cache.stride(0), key_cache.stride(1)
    a.vc_stride_block, a.vc_stride_head = value_cache.stride(0), value_cache.stride(1)
    a.num_blocks = key_cache.shape[0]
    if rot_mode == _lib.ROT_LAZY:
        if packed_block_table.dtype != torch.int64 or packed_block_table.stride(1) != 1:
            raise ValueError("the decode block table must be the packed int64 table")
        _require_cuda(packed_block_table)
        a.packed_block_table = packed_block_table.data_ptr()
        a.packed_stride = packed_block_table.stride(0)
    else:
        _i32(block_table, "block_table"); _i32(q_mask, "q_mask")
        _require_cuda(block_table, q_mask)
        if block_table.stride(1) != 1 or q_mask.stride(1) != 1 or q_mask.stride(0) != block_table.stride(0):
            raise ValueError("block_table and q_mask must share strides")
        a.block_table, a.q_mask = block_table.data_ptr(), q_mask.data_ptr()
        a.table_stride = block_table.stride(0)
    a.query_start_loc, a.seq_lens = query_start_loc.data_ptr(), seq_lens.data_ptr()
    lazy_u8 = _bool_u8(is_lazy)
    a.is_lazy = _ptr(lazy_u8)
    if alibi_slopes is not None:
        if alibi_slopes.dtype != torch.float32:
            raise ValueError("alibi_slopes must be float32")
        a.alibi_slopes = alibi_slopes.data_ptr()
    ks, vs = _scale(k_scale, query.device), _scale(v_scale, query.device)
    a.k_scale, a.v_scale = ks.data_ptr(), vs.data_ptr()
    if cos_sin_cache is not None:
        _require_cuda(cos_sin_cache)
        if cos_sin_cache.dtype not in _ACT or not cos_sin_cache.is_contiguous():
            raise ValueError("cos_sin_cache must be a contiguous f32/f16/bf16 tensor")
        a.cos_sin_cache = cos_sin_cache.data_ptr()
        a.cos_sin_rows = cos_sin_cache.shape[0]
        a.cos_sin_dtype = _ACT[cos_sin_cache.dtype]
    a.num_seqs = len(seq_lens)
    a.num_q_heads, a.num_kv_heads, a.head_dim = query.shape[1], key_cache.shape[1], query.shape[2]
    a.block_size, a.x = bs, x
    a.max_seq_len = int(max_seq_len) if max_seq_len is not None else 0
    a.q_dtype, a.kv_dtype = _ACT[query.dtype], kv_code
    a.rotary_dim = int(rotary_dim) if rotary_dim is not None else query.shape[2]
    a.sliding_window = int(sliding_window)
    a.rot_mode = rot_mode
    a.ignore_q_mask = int(bool(ignore_q_mask))
    a.sm_scale = float(sm_scale)
    a.kernel = _kernel_choice(kernel)
    if peer_out is not None:
        peer_out.fill(a.peer)
    if slot_mapping is not None:
        _require_cuda(key, value)
        if key.dtype != query.dtype or value.dtype != query.dtype or key.stride(2) != 1 or value.stride(2) != 1:
            raise ValueError("key / value must have the query's dtype and a contiguous last dimension")
        a.key, a.value = key.data_ptr(), value.data_ptr()
        a.k_stride_t, a.k_stride_h = key.stride(0), key.stride(1)
        a.v_stride_t, a.v_stride_h = value.stride(0), value.stride(1)
        a.slot_mapping = _slots(slot_mapping, query.shape[0])
    a.q_positions = _positions(positions)
    if rope_meta is not None:
        # in-kernel cos/sin from the rotary layer's parameters (keys of rope_meta_from_layer)
        a.compute_cos_sin = 1
        a.rope_type = int(rope_meta.get("ROPE_TYPE", 0))
        a.rope_base = float(rope_meta.get("BASE", 10000.0))
        a.rope_scaling_factor = float(rope_meta.get("SCALING_FACTOR", 1.0))
        a.rope_low_freq_factor = float(rope_meta.get("LOW_FACTOR", 1.0))
        a.rope_high_freq_factor = float(rope_meta.get("HIGH_FACTOR", 1.0))
        a.rope_orig_max_position = int(rope_meta.get("ORIG_MAX_POSITION", 8192))
    lib = _lib.load()
    need = lib.la_decode_workspace_bytes(C.byref(a))
    ws = _workspace(query.device, need)
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(query.device):
        rc = lib.la_decode_fwd(C.byref(a), torch.cuda.current_stream(query.device).cuda_stream)
    _lib.check(rc, "la_decode_fwd")


def _decode_rope_meta(rope_meta):
    """RoPE parameters for in-kernel cos/sin, or None to load them from the table
    (the reference's switch, lazy_attn/lazy/utils/variants.py:136-137)."""
    if not _env_flag("LAZY_DECODE_COMPUTE_COS_SIN"):
        return None
    if rope_meta is not None:
        return rope_meta
    return dict(ROPE_TYPE=0, BASE=10000.0, SCALING_FACTOR=1.0, LOW_FACTOR=1.0, HIGH_FACTOR=1.0,
                ORIG_MAX_POSITION=8192)


@torch.inference_mode()
def chunked_prefill_paged_decode(query, key, value, output, kv_cache_dtype, key_cache, value_cache,
                                 block_table, query_start_loc, seq_lens, max_seq_len,
                                 max_query_len, k_scale, v_scale, alibi_slopes=None,
                                 sliding_window=None, sm_scale=None, rotary_dim=None, freqs=None,
                                 cos_sin_cache=None, rope_meta=None, is_neox_style=True,
                                 is_lazy=None, lazy_variant=None, q_offset=None, q_mask=None,
                                 packed_block_table=None, kernel=None, peer_out=None, slot_mapping=None,
                                 positions=None):
    """One attention-layer call on a mixed batch: prefix-prefill for requests with
    more than one query token, paged decode for those with exactly one.

    Keeps the reference's quirks: the default ``sm_scale`` is
    ``1/sqrt(query.shape[1])`` (the head count), ``NO_LAZY=1`` clears
    ``is_lazy`` in place, and the decode kernel reads block ids from the packed
    table's high half, so ``packed_block_table`` is required for decode.  As in the
    reference (ops/chunked_prefill_paged_decode.py:146-155) the decode kernel loads
    cos/sin from ``cos_sin_cache`` unless ``LAZY_DECODE_COMPUTE_COS_SIN=1``, in which
    case it computes them from ``rope_meta`` (plain RoPE with base 10000 when that is
    missing, the reference's default); ``freqs`` is accepted and unused, as there.
    """
    if _env_flag("NO_LAZY") and is_lazy is not None:
        is_lazy.fill_(False)
    if sm_scale is None:
        sm_scale = 1.0 / (query.shape[1] ** 0.5)
    if sliding_window is None or sliding_window <= 0:
        sliding_window = 0
    if max_query_len > 1:
        context_attention_fwd(q=query, k=key, v=value, o=output, kv_cache_dtype=kv_cache_dtype,
                              k_cache=key_cache, v_cache=value_cache, b_loc=block_table,
                              b_start_loc=query_start_loc, b_seq_len=seq_lens,
                              max_seq_len=max_seq_len, max_input_len=max_query_len,
                              k_scale=k_scale, v_scale=v_scale, alibi_slopes=alibi_slopes,
                              sliding_window=sliding_window, sm_scale=sm_scale, skip_decode=True,
                              rotary_dim=rotary_dim, cos_sin_cache=cos_sin_cache,
                              is_neox_style=is_neox_style, is_lazy=is_lazy, q_offset=q_offset,
                              q_mask=q_mask, kernel=kernel, peer_out=peer_out,
                              packed_block_table=packed_block_table, slot_mapping=slot_mapping,
                              positions=positions)
    table = packed_block_table
    if table is None:
        # The reference would hand the kernel the plain table and unpack garbage
        # from it; refuse instead.
        raise ValueError("chunked_prefill_paged_decode needs packed_block_table for the decode kernel")
    _decode(query, output, kv_cache_dtype, key_cache, value_cache, query_start_loc, seq_lens,
            max_seq_len, k_scale, v_scale, alibi_slopes, sliding_window, sm_scale, rotary_dim,
            cos_sin_cache, is_lazy, table, None, None, _lib.ROT_LAZY,
            _env_flag("LAZY_DECODE_IGNORE_Q_MASK"), kernel, peer_out, key, value, slot_mapping, positions,
            _decode_rope_meta(rope_meta))


@torch.inference_mode()
def chunked_prefill_paged_decode_mepic(query, key, value, output, kv_cache_dtype, key_cache,
                                       value_cache, block_table, query_start_loc, seq_lens,
                                       max_seq_len, max_query_len, k_scale, v_scale,
                                       alibi_slopes=None, sliding_window=None, sm_scale=None,
                                       rotary_dim=None, cos_sin_cache=None, is_neox_style=True,
                                       q_offset=None, q_mask=None, is_mepic: bool = True,
                                       force_fp32_rotary: bool = False, kernel=None, peer_out=None,
                                       slot_mapping=None, positions=None):
    """Per-token rotation twin of :func:`chunked_prefill_paged_decode`: plain
    int32 block table and ``q_mask``; missing ``q_mask`` / ``q_offset`` mean zeros."""
    if sm_scale is None:
        sm_scale = 1.0 / (query.shape[1] ** 0.5)
    if sliding_window is None or sliding_window <= 0:
        sliding_window = 0
    if q_mask is None:
        q_mask = torch.zeros_like(block_table, dtype=torch.int32)
    if q_offset is None:
        q_offset = torch.zeros_like(block_table, dtype=torch.int32)
    if max_query_len > 1:
        context_attention_fwd_mepic(q=query, k=key, v=value, o=output,
                                    kv_cache_dtype=kv_cache_dtype, k_cache=key_cache,
                                    v_cache=value_cache, b_loc=block_table,
                                    b_start_loc=query_start_loc, b_seq_len=seq_lens,
                                    max_seq_len=max_seq_len, max_input_len=max_query_len,
                                    k_scale=k_scale, v_scale=v_scale, alibi_slopes=alibi_slopes,
                                    sliding_window=sliding_window, sm_scale=sm_scale,
                                    skip_decode=True, rotary_dim=rotary_dim,
                                    cos_sin_cache=cos_sin_cache, is_neox_style=is_neox_style,
                                    q_mask=q_mask, q_offset=q_offset, is_mepic=is_mepic,
                                    force_fp32_rotary=force_fp32_rotary, kernel=kernel,
                                    peer_out=peer_out, slot_mapping=slot_mapping, positions=positions)
    _decode(query, output, kv_cache_dtype, key_cache, value_cache, query_start_loc, seq_lens,
            max_seq_len, k_scale, v_scale, alibi_slopes, sliding_window, sm_scale, rotary_dim,
            cos_sin_cache, None, None, block_table, q_mask, _lib.ROT_MEPIC, False, kernel, peer_out,
            key, value, slot_mapping, positions)
