"""The C ABI library loads and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

from lazy_attention_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "lazy_attention_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(la_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = _lib.load()
    names = declared_symbols()
    assert "la_prefill_fwd" in names and "la_decode_fwd" in names
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(_lib.EXPORTS) <= set(names)


def test_version_and_error_text():
    lib = _lib.load()
    assert lib.la_version() == 101
    assert isinstance(_lib.last_error(), str)
    assert lib.la_launch_count() >= 0


def test_struct_sizes_match_header():
    # Compile-time layout is mirrored field by field; guard the totals against drift.
    assert ctypes.sizeof(_lib.LaPrefillArgs) % 8 == 0
    assert ctypes.sizeof(_lib.LaDecodeArgs) % 8 == 0
    lib = _lib.load()
    assert lib.la_sizeof_prefill_args() == ctypes.sizeof(_lib.LaPrefillArgs)
    assert lib.la_sizeof_decode_args() == ctypes.sizeof(_lib.LaDecodeArgs)


def test_null_arguments_are_refused_without_a_gpu():
    lib = _lib.load()
    assert lib.la_prefill_fwd(None, None) == _lib.LA_ERR_INVALID_ARGUMENT
    assert "null" in _lib.last_error()
    assert lib.la_decode_fwd(None, None) == _lib.LA_ERR_INVALID_ARGUMENT
    assert lib.la_pack_block_table(None, None, None, None, None, 1, 1, 1, 1, None) == _lib.LA_ERR_INVALID_ARGUMENT
    assert lib.la_build_cos_sin_table(None, 0, 4, 8, 1e4, 0, 1.0, 1.0, 1.0, 8192, None) == _lib.LA_ERR_INVALID_ARGUMENT
    assert lib.la_peer_barrier(None, 2, 0, None) == _lib.LA_ERR_INVALID_ARGUMENT
    one = (ctypes.c_void_p * 2)(0x1000, None)
    assert lib.la_peer_barrier(one, 2, 0, None) == _lib.LA_ERR_INVALID_ARGUMENT   # a rank without a signal buffer
    assert lib.la_peer_barrier(one, 1, 1, None) == _lib.LA_ERR_INVALID_ARGUMENT   # rank outside the job
    assert lib.la_peer_barrier(one, _lib.LA_MAX_PEERS + 1, 0, None) == _lib.LA_ERR_INVALID_ARGUMENT


def _split_prefill_args():
    """A call the tensor-core kernel accepts and splits over the KV range (64 CTAs of one row
    block each against 148 SMs); the pointers are made up and never dereferenced on the host."""
    a = _lib.LaPrefillArgs()
    a.q = a.k = a.v = a.out = 0x10000
    a.k_cache = a.v_cache = 0x20000
    a.block_table = a.query_start_loc = a.seq_lens = 0x30000
    a.q_stride_t, a.q_stride_h = 32 * 128, 128
    a.k_stride_t, a.k_stride_h = 8 * 128, 128
    a.v_stride_t, a.v_stride_h = 8 * 128, 128
    a.o_stride_t, a.o_stride_h = 32 * 128, 128
    a.kc_stride_block = a.vc_stride_block = 8 * 128 * 16
    a.kc_stride_head = a.vc_stride_head = 128 * 16
    a.num_blocks, a.table_stride = 4096, 520
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = 8, 32, 8, 128
    a.block_size, a.x, a.max_query_len, a.max_seq_len = 16, 8, 64, 8192
    a.q_dtype = a.kv_dtype = _lib.DTYPE_BF16
    a.rotary_dim, a.rot_mode, a.sm_scale = 128, _lib.ROT_LAZY, 0.088
    return a


def test_missing_workspace_is_an_error_not_a_slow_path():
    """Automatic kernel selection never falls back to the general kernel because the
    split-KV workspace is absent or short: the call fails with LA_ERR_WORKSPACE and says how
    many bytes it needs (checked before anything touches the device, so it runs without a GPU)."""
    lib = _lib.load()
    a = _split_prefill_args()
    need = lib.la_prefill_workspace_bytes(ctypes.byref(a))
    assert need > 0, "pick a call that splits"
    for kernel in (_lib.KERNEL_AUTO, _lib.KERNEL_TENSOR):
        a.kernel = kernel
        a.workspace, a.workspace_bytes = None, 0
        assert lib.la_prefill_fwd(ctypes.byref(a), None) == _lib.LA_ERR_WORKSPACE
        assert str(need) in _lib.last_error()
        a.workspace, a.workspace_bytes = 0x40000, need - 1
        assert lib.la_prefill_fwd(ctypes.byref(a), None) == _lib.LA_ERR_WORKSPACE
    assert lib.la_prefill_fwd_noalloc(None, None) == _lib.LA_ERR_INVALID_ARGUMENT


def test_a_batch_beyond_the_launch_grid_is_refused():
    """More requests x splits than a grid dimension holds: a status code with the numbers, before
    anything touches the device."""
    lib = _lib.load()
    a = _split_prefill_args()
    a.batch = 70000
    a.kernel = _lib.KERNEL_TENSOR
    assert lib.la_prefill_fwd(ctypes.byref(a), None) == _lib.LA_ERR_UNSUPPORTED
    assert "70000" in _lib.last_error() and "65535" in _lib.last_error()


def test_patch_in_binds_what_the_reference_backend_passes():
    """The keyword sets the reference backend passes to its two operators, and the modules it
    imports them from, were read from its source when the fixtures were made
    (tests/golden/backend_keywords.json, from lazy_attn/lazy/attention/backends/triton_attn.py):
    the replacement operators must bind exactly those calls, so a rename in the reference
    shows up when the fixture is regenerated."""
    import inspect
    import json
    import types
    from lazy_attention_b200 import vllm_patch
    import lazy_attention_b200 as la

    rec = json.loads((ROOT / "tests" / "golden" / "backend_keywords.json").read_text())
    assert set(rec["imports"]) == {"chunked_prefill_paged_decode", "chunked_prefill_paged_decode_old"}
    assert rec["imports"]["chunked_prefill_paged_decode"].endswith("ops.chunked_prefill_paged_decode")
    assert rec["imports"]["chunked_prefill_paged_decode_old"].endswith("old_ops.chunked_prefill_paged_decode")
    backend = types.ModuleType("fake_triton_attn")
    previous = vllm_patch.install(backend)
    for name, extra in rec["extra"].items():
        fn = getattr(backend, name)
        inspect.signature(fn).bind(**{k: None for k in rec["common"] + extra})
    assert backend.chunked_prefill_paged_decode is la.chunked_prefill_paged_decode
    assert backend.chunked_prefill_paged_decode_old is la.chunked_prefill_paged_decode_mepic
    vllm_patch.uninstall(previous, backend)


def test_patch_in_rebinds_backend_and_accepts_its_keywords():
    """The two names the reference backend calls are rebound, and the replacement
    functions accept exactly the keyword sets the backend passes
    (lazy_attn/lazy/attention/backends/triton_attn.py:146-187)."""
    import inspect
    import types
    from lazy_attention_b200 import vllm_patch
    import lazy_attention_b200 as la

    backend = types.ModuleType("fake_triton_attn")
    sentinel = object()
    backend.chunked_prefill_paged_decode = sentinel
    previous = vllm_patch.install(backend)
    assert backend.chunked_prefill_paged_decode is la.chunked_prefill_paged_decode
    assert backend.chunked_prefill_paged_decode_old is la.chunked_prefill_paged_decode_mepic
    common = ["query", "key", "value", "output", "kv_cache_dtype", "key_cache", "value_cache", "block_table",
              "query_start_loc", "seq_lens", "max_seq_len", "max_query_len", "k_scale", "v_scale", "alibi_slopes",
              "sliding_window", "sm_scale", "cos_sin_cache", "rotary_dim", "is_neox_style"]
    lazy_kw = common + ["freqs", "rope_meta", "is_lazy", "lazy_variant", "q_offset", "q_mask", "packed_block_table"]
    mepic_kw = common + ["q_offset", "q_mask", "is_mepic", "force_fp32_rotary"]
    inspect.signature(backend.chunked_prefill_paged_decode).bind(**{k: None for k in lazy_kw})
    inspect.signature(backend.chunked_prefill_paged_decode_old).bind(**{k: None for k in mepic_kw})
    vllm_patch.uninstall(previous, backend)
    assert backend.chunked_prefill_paged_decode is sentinel
    assert not hasattr(backend, "chunked_prefill_paged_decode_old")
