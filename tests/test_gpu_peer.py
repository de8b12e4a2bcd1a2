"""The fused output gather on ONE GPU: the "ranks'" buffers are all local.

The kernels only see pointers, strides, a head offset and a row map (``LaPeerOut``), so every
store path of the gather -- the tensor-core kernel's epilogue through shared memory, the
split-KV merge kernel, the decode kernels -- can be checked without a second device: rows
written into each buffer must equal, bit for bit, what the same call writes into ``out``, and
nothing else in the buffers may change.  The end-of-step signal kernel is run with one rank.
Two real GPUs are covered by test_gpu_multi.py.
"""
import ctypes as C

import pytest
import torch

import util
import lazy_attention_b200 as la
from lazy_attention_b200 import _lib, sharding, synth

pytestmark = pytest.mark.gpu

POOL = [100, 64, 33, 250, 16, 129, 700]


class LocalPeers:
    """What the operators need from ``sharding.PeerOutput`` (``fill``), over local tensors."""

    def __init__(self, buffers, head_offset=0, rows=None):
        self.buffers, self.head_offset, self.rows = buffers, head_offset, rows

    def fill(self, peer):
        for r, t in enumerate(self.buffers):
            peer.out[r] = t.data_ptr()
        peer.num_peers = len(self.buffers)
        peer.head_offset = self.head_offset
        peer.stride_t, peer.stride_h = self.buffers[0].stride(0), self.buffers[0].stride(1)
        peer.rows = self.rows.data_ptr() if self.rows is not None else None


def _check(case, op, kernel, nbuf=3):
    g = case["geom"]
    T, H, D = case["num_tokens"], g.num_q_heads, g.head_dim
    want = util.run_cuda(case, op, kernel=kernel)
    # buffers of a job with twice the heads and a few more rows, rows permuted
    perm = torch.randperm(T + 5, generator=torch.Generator().manual_seed(T))[:T].to(torch.int32)
    dtype = case["q"].dtype
    bufs = [torch.full((T + 5, 2 * H, D), 7.0, dtype=dtype, device="cuda") for _ in range(nbuf)]
    peers = LocalPeers(bufs, head_offset=H, rows=perm.cuda())
    util.run_cuda(case, op, kernel=kernel, peer_out=peers)
    rows = perm.long()
    for i, b in enumerate(bufs):
        b = b.float().cpu()
        assert torch.equal(b[rows][:, H:], want), f"buffer {i}: gathered rows differ from the plain call"
        assert bool((b[:, :H] == 7.0).all()), f"buffer {i}: heads outside the rank's range were touched"
        rest = torch.ones(T + 5, dtype=torch.bool)
        rest[rows] = False
        assert bool((b[rest] == 7.0).all()), f"buffer {i}: rows outside the map were touched"


@pytest.mark.parametrize("splits", ["1", "3"])
@pytest.mark.parametrize("geom", [synth.GEOM_1B, synth.GEOM_8B], ids=["d64", "d128"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_prefill_gather_rows(splits, geom, dtype, monkeypatch):
    """splits=1: the attention kernel's own epilogue stores the rows; 3: the merge kernel does."""
    monkeypatch.setenv("LAZY_ATTN_B200_PREFILL_SPLITS", splits)
    reqs = [dict(docs=[2, 0, 1], qlen=37), dict(docs=[3, 6, 5], qlen=300), dict(docs=[1, 4], qlen=129),
            dict(docs=[0], qlen=16, lazy=False), dict(docs=[], qlen=64)]
    case = synth.build_prefill(geom, dtype, POOL, reqs, seed=31, variant="lazy", device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    _check(case, "lazy_prefill", "tensor")


def test_prefill_gather_rows_fp8_cache(monkeypatch):
    """fp8 caches (pages converted in shared memory by the staging warps) share the epilogue."""
    monkeypatch.setenv("LAZY_ATTN_B200_PREFILL_SPLITS", "1")
    reqs = [dict(docs=[2, 0, 1], qlen=200), dict(docs=[3, 6], qlen=257)]
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, POOL, reqs, seed=32, variant="lazy", device="cuda",
                               kv_dtype="fp8_e4m3", k_scale=0.11, v_scale=0.07)
    case["packed_block_table"] = util.pack_host(case).cuda()
    _check(case, "lazy_prefill", "tensor")


@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
def test_decode_gather_rows(kv):
    docs = [[512, 1024], [256], [2048, 160], [512], [4096, 4096, 1024]]
    scales = dict(k_scale=0.1, v_scale=0.2) if "fp8" in kv else {}
    case = synth.build_decode(synth.GEOM_8B, torch.bfloat16, docs, seed=33, device="cuda", kv_dtype=kv, **scales)
    case["packed_block_table"] = util.pack_host(case).cuda()
    _check(case, "lazy_op", "tensor")


def test_signal_kernel_one_rank():
    """One rank: the kernel announces to itself and returns; the round counter advances per call."""
    lib = _lib.load()
    sig = C.c_void_p()
    assert lib.la_peer_alloc(_lib.LA_PEER_SIGNAL_BYTES, C.byref(sig)) == 0, _lib.last_error()
    try:
        arr = (C.c_void_p * 1)(sig.value)
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            assert lib.la_peer_barrier(arr, 1, 0, stream) == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert la.device_status() == 0
        words = sharding._as_tensor(sig.value, (_lib.LA_PEER_SIGNAL_BYTES // 2,), torch.float16,
                                    torch.device("cuda", torch.cuda.current_device())).view(torch.int32).cpu()
        assert int(words[0]) == 3 and int(words[32]) == 3
        assert int(words.abs().sum()) == 6, "only the rank's own slot and the round counter are written"
    finally:
        lib.la_peer_free(sig)


def test_signal_kernel_gives_up_on_a_rank_that_never_arrives(monkeypatch):
    """Rank 0 of 2 with a second signal buffer nobody writes: the wait runs out after the (shortened)
    limit, the kernel returns, the status word names the missing rank, and the device stays usable."""
    monkeypatch.setenv("LAZY_ATTN_B200_BARRIER_LIMIT_MS", "200")
    lib = _lib.load()
    mine, silent = C.c_void_p(), C.c_void_p()
    assert lib.la_peer_alloc(_lib.LA_PEER_SIGNAL_BYTES, C.byref(mine)) == 0, _lib.last_error()
    assert lib.la_peer_alloc(_lib.LA_PEER_SIGNAL_BYTES, C.byref(silent)) == 0, _lib.last_error()
    try:
        assert la.device_status() == 0
        arr = (C.c_void_p * 2)(mine.value, silent.value)
        assert lib.la_peer_barrier(arr, 2, 0, torch.cuda.current_stream().cuda_stream) == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert lib.la_check_device() == _lib.LA_ERR_DEVICE_STATUS
        assert "301" in _lib.last_error()
        assert la.device_status() == 0, "reading the status clears it"
        # the context is intact: a one-rank round still completes
        one = (C.c_void_p * 1)(mine.value)
        assert lib.la_peer_barrier(one, 1, 0, torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        assert la.device_status() == 0
        x = torch.arange(8, device="cuda")
        assert int(x.sum()) == 28
    finally:
        lib.la_peer_free(mine)
        lib.la_peer_free(silent)
