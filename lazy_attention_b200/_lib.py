"""ctypes binding of ``liblazy_attention_b200.so`` (the C ABI in
``include/lazy_attention_b200.h``).  Loading fails loudly: there is no Python
or CPU stand-in for the CUDA library."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "liblazy_attention_b200.so"

LA_OK = 0
LA_ERR_INVALID_ARGUMENT = -1
LA_ERR_UNSUPPORTED = -2
LA_ERR_CUDA = -3
LA_ERR_WORKSPACE = -4
LA_ERR_DEVICE_STATUS = -5

DTYPE_F32, DTYPE_F16, DTYPE_BF16, DTYPE_FP8_E4M3, DTYPE_FP8_E5M2 = range(5)
ROT_LAZY, ROT_MEPIC = 0, 1
KERNEL_AUTO, KERNEL_GENERAL, KERNEL_TENSOR = 0, 1, 2

EXPORTS = (
    "la_prefill_fwd", "la_decode_fwd", "la_prefill_workspace_bytes",
    "la_decode_workspace_bytes", "la_pack_block_table",
    "la_build_cos_sin_table", "la_last_error", "la_version", "la_launch_count",
    "la_sizeof_prefill_args", "la_sizeof_decode_args", "la_device_status",
    "la_prefill_fwd_noalloc", "la_write_paged_cache",
    "la_check_device", "la_peer_alloc", "la_peer_export", "la_peer_open", "la_peer_close", "la_peer_free", "la_peer_barrier",
)


LA_MAX_PEERS = 8
LA_PEER_SIGNAL_BYTES = 256


class LaPeerOut(C.Structure):
    _fields_ = [
        ("out", C.c_void_p * LA_MAX_PEERS), ("num_peers", C.c_int32), ("head_offset", C.c_int32),
        ("stride_t", C.c_int64), ("stride_h", C.c_int64), ("rows", C.c_void_p),
    ]


class LaPrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
        ("k_stride_t", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_t", C.c_int64), ("v_stride_h", C.c_int64),
        ("o_stride_t", C.c_int64), ("o_stride_h", C.c_int64),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("kc_stride_block", C.c_int64), ("kc_stride_head", C.c_int64),
        ("vc_stride_block", C.c_int64), ("vc_stride_head", C.c_int64),
        ("num_blocks", C.c_int64),
        ("block_table", C.c_void_p), ("q_offset", C.c_void_p), ("q_mask", C.c_void_p),
        ("table_stride", C.c_int64),
        ("query_start_loc", C.c_void_p), ("seq_lens", C.c_void_p), ("is_lazy", C.c_void_p),
        ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("cos_sin_cache", C.c_void_p), ("cos_sin_rows", C.c_int64),
        ("cos_sin_dtype", C.c_int32), ("batch", C.c_int32),
        ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("block_size", C.c_int32), ("x", C.c_int32), ("max_query_len", C.c_int32),
        ("max_seq_len", C.c_int32),
        ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("rotary_dim", C.c_int32),
        ("sliding_window", C.c_int32), ("skip_decode", C.c_int32),
        ("rot_mode", C.c_int32), ("is_mepic", C.c_int32),
        ("sm_scale", C.c_float), ("kernel", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("peer", LaPeerOut),
        ("packed_block_table", C.c_void_p), ("packed_stride", C.c_int64),
        ("slot_mapping", C.c_void_p),
        ("q_positions", C.c_void_p),
    ]


class LaDecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p),
        ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
        ("o_stride_t", C.c_int64), ("o_stride_h", C.c_int64),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("kc_stride_block", C.c_int64), ("kc_stride_head", C.c_int64),
        ("vc_stride_block", C.c_int64), ("vc_stride_head", C.c_int64),
        ("num_blocks", C.c_int64),
        ("packed_block_table", C.c_void_p), ("packed_stride", C.c_int64),
        ("block_table", C.c_void_p), ("q_mask", C.c_void_p), ("table_stride", C.c_int64),
        ("query_start_loc", C.c_void_p), ("seq_lens", C.c_void_p), ("is_lazy", C.c_void_p),
        ("alibi_slopes", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("cos_sin_cache", C.c_void_p), ("cos_sin_rows", C.c_int64),
        ("cos_sin_dtype", C.c_int32), ("num_seqs", C.c_int32),
        ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("block_size", C.c_int32), ("x", C.c_int32), ("max_seq_len", C.c_int32),
        ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("rotary_dim", C.c_int32),
        ("sliding_window", C.c_int32), ("rot_mode", C.c_int32),
        ("ignore_q_mask", C.c_int32), ("sm_scale", C.c_float), ("kernel", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("peer", LaPeerOut),
        ("key", C.c_void_p), ("value", C.c_void_p),
        ("k_stride_t", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_t", C.c_int64), ("v_stride_h", C.c_int64),
        ("slot_mapping", C.c_void_p),
        ("q_positions", C.c_void_p),
        ("compute_cos_sin", C.c_int32), ("rope_type", C.c_int32),
        ("rope_base", C.c_float), ("rope_scaling_factor", C.c_float),
        ("rope_low_freq_factor", C.c_float), ("rope_high_freq_factor", C.c_float),
        ("rope_orig_max_position", C.c_int32), ("reserved0", C.c_int32),
    ]


class LaWriteCacheArgs(C.Structure):
    _fields_ = [
        ("key", C.c_void_p), ("value", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("slot_mapping", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("k_stride_t", C.c_int64), ("k_stride_h", C.c_int64), ("v_stride_t", C.c_int64), ("v_stride_h", C.c_int64),
        ("kc_stride_block", C.c_int64), ("kc_stride_head", C.c_int64),
        ("vc_stride_block", C.c_int64), ("vc_stride_head", C.c_int64),
        ("num_tokens", C.c_int64),
        ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("block_size", C.c_int32), ("x", C.c_int32),
        ("dtype", C.c_int32), ("kv_dtype", C.c_int32),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m lazy_attention_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    lib.la_prefill_fwd.argtypes = [C.POINTER(LaPrefillArgs), C.c_void_p]
    lib.la_prefill_fwd.restype = C.c_int
    lib.la_prefill_fwd_noalloc.argtypes = [C.POINTER(LaPrefillArgs), C.c_void_p]
    lib.la_prefill_fwd_noalloc.restype = C.c_int
    lib.la_write_paged_cache.argtypes = [C.POINTER(LaWriteCacheArgs), C.c_void_p]
    lib.la_write_paged_cache.restype = C.c_int
    lib.la_decode_fwd.argtypes = [C.POINTER(LaDecodeArgs), C.c_void_p]
    lib.la_decode_fwd.restype = C.c_int
    lib.la_prefill_workspace_bytes.argtypes = [C.POINTER(LaPrefillArgs)]
    lib.la_prefill_workspace_bytes.restype = C.c_size_t
    lib.la_decode_workspace_bytes.argtypes = [C.POINTER(LaDecodeArgs)]
    lib.la_decode_workspace_bytes.restype = C.c_size_t
    lib.la_pack_block_table.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_int32, C.c_int32, C.c_int64,
                                        C.c_int64, C.c_void_p]
    lib.la_pack_block_table.restype = C.c_int
    lib.la_build_cos_sin_table.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                           C.c_double, C.c_int32, C.c_double, C.c_double,
                                           C.c_double, C.c_int64, C.c_void_p]
    lib.la_build_cos_sin_table.restype = C.c_int
    lib.la_last_error.argtypes = []
    lib.la_last_error.restype = C.c_char_p
    lib.la_version.argtypes = []
    lib.la_version.restype = C.c_int
    lib.la_launch_count.argtypes = []
    lib.la_launch_count.restype = C.c_int64
    lib.la_device_status.argtypes = []
    lib.la_device_status.restype = C.c_int
    lib.la_check_device.argtypes = []
    lib.la_check_device.restype = C.c_int
    lib.la_peer_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
    lib.la_peer_export.argtypes = [C.c_void_p, C.c_char_p]
    lib.la_peer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.la_peer_close.argtypes = [C.c_void_p]
    lib.la_peer_free.argtypes = [C.c_void_p]
    lib.la_peer_barrier.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_void_p]
    for fn in (lib.la_peer_alloc, lib.la_peer_export, lib.la_peer_open, lib.la_peer_close, lib.la_peer_free,
               lib.la_peer_barrier):
        fn.restype = C.c_int
    lib.la_sizeof_prefill_args.restype = C.c_size_t
    lib.la_sizeof_decode_args.restype = C.c_size_t
    if (lib.la_sizeof_prefill_args() != C.sizeof(LaPrefillArgs)
            or lib.la_sizeof_decode_args() != C.sizeof(LaDecodeArgs)):
        raise RuntimeError("liblazy_attention_b200.so was built from a different header; rebuild it")
    _lib = lib
    return lib


def last_error() -> str:
    return load().la_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    """Map a C-ABI status to the Python exception the reference raises."""
    if rc == LA_OK:
        return
    msg = f"{what}: {last_error()}"
    if rc == LA_ERR_INVALID_ARGUMENT:
        raise ValueError(msg)
    if rc == LA_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"{msg} (status {rc})")
