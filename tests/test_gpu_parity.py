"""GPU parity: the CUDA library, called through the C ABI, against the golden
fixtures (reference kernel outputs) and against the CPU oracle on seeded inputs.

Tolerances: float32 2e-5 abs / 1e-5 rel against the reference fixtures;
bf16 / fp16 max-abs 2e-2, rel 1e-2 against the float32 oracle; fp8 KV 5e-2 abs
against an oracle that dequantises the same stored bytes.  Integer results
(packed table) are compared bit for bit.
"""
import numpy as np
import pytest
import torch

import util
from lazy_attention_b200 import synth
from oracle import lazy_oracle as oracle

pytestmark = pytest.mark.gpu

F32 = dict(atol=2e-5, rtol=1e-5)
HALF = dict(atol=2e-2, rtol=1e-2)
FP8 = dict(atol=5e-2, rtol=1e-2)

GOLDEN_CASES = [
    ("lazy_prefill_small", "lazy_prefill", dict(skip_decode=True)),
    ("lazy_mixed_small", "lazy_op", {}),
    ("mepic_mixed_small", "mepic_op", dict(is_mepic=True)),
    ("mepic_off_mixed_small", "mepic_op", dict(is_mepic=False)),
    ("lazy_decode_fp8_small", "lazy_op", {}),
    ("plain_prefill_fp8_small", "lazy_prefill", {}),
    ("lazy_mixed_window_small", "lazy_op", {}),
    ("lazy_decode_alibi_small", "lazy_op", {}),
    ("lazy_mixed_bs8_small", "lazy_op", {}),
]


@pytest.mark.parametrize("name,op,kw", GOLDEN_CASES, ids=[c[0] for c in GOLDEN_CASES])
def test_general_kernel_matches_reference_fixtures(name, op, kw):
    case = util.load_golden(name)
    got = util.run_cuda(case, op, kernel="general", **kw)
    util.assert_close(got, case["out"], what=name, **F32)


@pytest.mark.parametrize("variant", ["lazy", "mepic"])
def test_first_config_fp32(variant):
    z = np.load(util.GOLDEN / f"c1_{variant}.npz")
    case = synth.config_c1(variant=variant)
    case["packed_block_table"] = util.pack_host(case)
    op = "lazy_prefill" if variant == "lazy" else "mepic_op"
    got = util.run_cuda(case, op, kernel="general")
    heads = [int(h) for h in z["heads"]]
    util.assert_close(got[:, heads], torch.from_numpy(z["out_heads"]), atol=1e-5, rtol=1e-5,
                      what=f"c1 {variant} vs reference kernel")
    util.assert_close(got, util.run_oracle(case, op), atol=1e-5, rtol=1e-5, what=f"c1 {variant} vs oracle")


POOL = [100, 64, 33, 250, 16, 129]
MIXED = [dict(docs=[2, 0, 1], qlen=37), dict(docs=[3, 1, 5], qlen=130), dict(docs=[0], qlen=16, lazy=False),
         dict(docs=[1, 2, 4], qlen=1), dict(docs=[4, 3], qlen=1), dict(docs=[2], qlen=1, lazy=False),
         dict(docs=[], qlen=20)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("geom", [synth.GEOM_1B, synth.GEOM_8B], ids=["d64", "d128"])
@pytest.mark.parametrize("variant", ["lazy", "mepic"])
@pytest.mark.parametrize("kernel", ["general", "auto"])
def test_half_precision_mixed_batch(dtype, geom, variant, kernel):
    case = synth.build_prefill(geom, dtype, POOL, MIXED, seed=3, variant=variant, device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    op = "lazy_op" if variant == "lazy" else "mepic_op"
    got = util.run_cuda(case, op, kernel=kernel)
    util.assert_close(got, util.run_oracle(case, op), what=f"{variant} {dtype} {kernel}", **HALF)


@pytest.mark.parametrize("kernel", ["general", "auto"])
@pytest.mark.parametrize("kv", ["fp8_e4m3", "fp8_e5m2"])
def test_fp8_cache_bf16_query(kernel, kv):
    reqs = [dict(docs=[3, 1, 5], qlen=1), dict(docs=[0, 2], qlen=1), dict(docs=[1], qlen=1, lazy=False),
            dict(docs=[4, 0], qlen=40), dict(docs=[5], qlen=9, lazy=False)]
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, POOL, reqs, seed=4, device="cuda",
                               kv_dtype=kv, k_scale=0.11, v_scale=0.07)
    case["packed_block_table"] = util.pack_host(case).cuda()
    got = util.run_cuda(case, "lazy_op", kernel=kernel)
    util.assert_close(got, util.run_oracle(case, "lazy_op"), what=f"fp8 {kv} {kernel}", **FP8)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("geom", [synth.GEOM_1B, synth.GEOM_8B], ids=["d64", "d128"])
@pytest.mark.parametrize("variant", ["lazy", "mepic"])
@pytest.mark.parametrize("kv", ["fp8_e4m3", "fp8_e5m2"])
def test_fp8_cache_tensor_core_prefill(dtype, geom, variant, kv):
    """fp8 caches through the tensor-core prefill kernel (pages converted to fp16
    and rotated while they are staged), against the oracle and the general kernel."""
    case = synth.build_prefill(geom, dtype, POOL, MIXED, seed=6, variant=variant, device="cuda",
                               kv_dtype=kv, k_scale=0.11, v_scale=0.07)
    case["packed_block_table"] = util.pack_host(case).cuda()
    op = "lazy_prefill" if variant == "lazy" else "mepic_prefill"
    got = util.run_cuda(case, op, kernel="tensor")
    util.assert_close(got, util.run_oracle(case, op), what=f"fp8 {kv} tensor {variant}", **FP8)
    util.assert_close(got, util.run_cuda(case, op, kernel="general"), what="tensor vs general", **FP8)


@pytest.mark.parametrize("heads", [(8, 8), (16, 2), (4, 4), (32, 16)], ids=["mha8", "g8", "mha4", "g2"])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("variant", ["lazy", "mepic"])
def test_other_head_groupings(heads, head_dim, variant):
    """Query heads per KV head other than the 4 of the BASELINE geometries (1, 2, 8),
    mixed prefill + decode batch, tensor-core / split-KV kernels against the oracle."""
    geom = synth.Geometry(heads[0], heads[1], head_dim)
    case = synth.build_prefill(geom, torch.bfloat16, POOL, MIXED, seed=8, variant=variant, device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    op = "lazy_op" if variant == "lazy" else "mepic_op"
    got = util.run_cuda(case, op, kernel="tensor")
    util.assert_close(got, util.run_oracle(case, op), what=f"{heads} d{head_dim} {variant}", **HALF)


@pytest.mark.parametrize("kernel", ["general", "tensor"])
def test_strided_views_of_a_fused_qkv_tensor(kernel):
    """q, k and v are column slices of one [T, (Hq + 2 Hkv) D] projection output (how
    the engine hands them over) and the output is a slice of a wider buffer: strides,
    not shapes, locate the rows."""
    geom = synth.GEOM_8B
    case = synth.build_prefill(geom, torch.bfloat16, POOL, MIXED, seed=12, device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    T, Hq, Hkv, D = case["num_tokens"], geom.num_q_heads, geom.num_kv_heads, geom.head_dim
    want = util.run_oracle(case, "lazy_op")
    fused = torch.zeros(T + 1, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16, device="cuda")
    fused[:T, :Hq * D] = case["q"][:T].reshape(T, -1)
    fused[:T, Hq * D:(Hq + Hkv) * D] = case["k"].reshape(T, -1)
    fused[:T, (Hq + Hkv) * D:] = case["v"].reshape(T, -1)
    strided = dict(case)
    strided["q"] = fused[:, :Hq * D].view(T + 1, Hq, D)
    strided["k"] = fused[:T, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    strided["v"] = fused[:T, (Hq + Hkv) * D:].view(T, Hkv, D)
    assert not strided["q"].is_contiguous()
    import lazy_attention_b200 as la
    wide = torch.zeros(T, Hq + 3, D + 8, dtype=torch.bfloat16, device="cuda")
    out = wide[:, 2:2 + Hq, :D]
    la.chunked_prefill_paged_decode(
        strided["q"], strided["k"], strided["v"], out, kv_cache_dtype="auto", key_cache=case["k_cache"],
        value_cache=case["v_cache"], block_table=case["block_table"], query_start_loc=case["query_start_loc"],
        seq_lens=case["seq_lens"], max_seq_len=case["max_seq_len"], max_query_len=case["max_query_len"],
        k_scale=case["k_scale"], v_scale=case["v_scale"], sm_scale=case["sm_scale"],
        cos_sin_cache=case["cos_sin_cache"], is_lazy=case["is_lazy"], q_offset=case["q_offset"],
        q_mask=case["q_mask"], packed_block_table=case["packed_block_table"], kernel=kernel)
    torch.cuda.synchronize()
    assert la.device_status() == 0
    util.assert_close(out.float().cpu(), want, what=f"strided views {kernel}", **HALF)
    assert float(wide[:, :2].abs().max()) == 0.0 and float(wide[:, :, D:].abs().max()) == 0.0, "wrote outside the view"


def test_many_short_requests():
    """64 requests with 0..3 short documents and 1..24 new tokens each."""
    import numpy as np
    rng = np.random.default_rng(3)
    pool = [16, 17, 31, 48, 5, 64]
    reqs = [dict(docs=[int(d) for d in rng.integers(0, len(pool), size=int(rng.integers(0, 4)))],
                 qlen=int(rng.integers(1, 25)), lazy=bool(rng.integers(0, 4) > 0)) for _ in range(64)]
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, pool, reqs, seed=13, device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    want = util.run_oracle(case, "lazy_op")
    for kernel in ("tensor", "general"):
        util.assert_close(util.run_cuda(case, "lazy_op", kernel=kernel), want, what=f"short requests {kernel}", **HALF)


@pytest.mark.parametrize("kernel", ["general", "auto"])
def test_second_config_bf16(kernel):
    """BASELINE config 2 at full size: 1B geometry, bf16, 10x512 cached tokens, 128 new."""
    case = synth.config_c2(device="cuda")
    got = util.run_cuda(case, "lazy_prefill", kernel=kernel)
    util.assert_close(got, util.run_oracle(case, "lazy_prefill"), what=f"c2 {kernel}", **HALF)


@pytest.mark.parametrize("kernel", ["general", "auto"])
def test_decode_zero_offset_keeps_previous_rotation(kernel):
    """Pages appended after the query page carry q_offset 0, which means "keep the
    rotation in force" (reference decode kernel); also covers a first page with 0."""
    geom = synth.GEOM_1B
    case = synth.build_decode(geom, torch.bfloat16, [[40, 100], [64], [200, 31, 5]], seed=9, device="cuda")
    # grow every sequence by two pages of generated tokens with zero metadata
    extra = 2 * geom.block_size
    nb = case["k_cache"].shape[0]
    bt = case["block_table"].cpu()
    S, cols = bt.shape
    new_bt = torch.zeros(S, cols + 2, dtype=torch.int32)
    new_off = torch.zeros(S, cols + 2, dtype=torch.int32)
    new_msk = torch.zeros(S, cols + 2, dtype=torch.int32)
    new_bt[:, :cols] = bt
    new_off[:, :cols] = case["q_offset"].cpu()
    new_msk[:, :cols] = case["q_mask"].cpu()
    seq = case["seq_lens"].cpu()
    for s in range(S):
        pages = (int(seq[s]) + geom.block_size - 1) // geom.block_size
        new_bt[s, pages:pages + 2] = torch.tensor([(7 * s + 1) % nb, (7 * s + 2) % nb])
    new_off[1, 0] = 0  # a leading zero offset: nothing to keep yet -> no rotation
    case["block_table"], case["q_offset"], case["q_mask"] = new_bt.cuda(), new_off.cuda(), new_msk.cuda()
    case["seq_lens"] = (seq + extra - 3).to(torch.int32).cuda()
    case["max_seq_len"] = int(case["seq_lens"].max())
    case["packed_block_table"] = util.pack_host(case).cuda()
    got = util.run_cuda(case, "lazy_op", kernel=kernel)
    util.assert_close(got, util.run_oracle(case, "lazy_op"), what="zero offsets", **HALF)


@pytest.mark.parametrize("geom", [synth.GEOM_1B, synth.GEOM_8B], ids=["d64", "d128"])
@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_decode_split_kv_long_context(geom, kv, dtype):
    """Decode over contexts long enough for several KV splits and ragged tails:
    documents with padding, a plain (non-rotating) sequence, a very short one."""
    docs = [[512] * 9, [500, 17, 1023, 256], [16], [700, 700, 700, 700, 700, 3], [33] * 20, [4096, 1]]
    flags = [True, True, True, True, False, True]
    ks, vs = (0.09, 0.13) if "fp8" in kv else (1.0, 1.0)
    case = synth.build_decode(geom, dtype, docs, seed=21, device="cuda", kv_dtype=kv, k_scale=ks,
                              v_scale=vs, lazy_flags=flags)
    got = util.run_cuda(case, "lazy_op", kernel="tensor")
    want = util.run_oracle(case, "lazy_op")
    util.assert_close(got, want, what=f"split-KV decode {kv}", **(FP8 if "fp8" in kv else HALF))
    general = util.run_cuda(case, "lazy_op", kernel="general")
    util.assert_close(got, general, what="split-KV vs general kernel", **(FP8 if "fp8" in kv else HALF))


@pytest.mark.parametrize("geom", [synth.GEOM_1B, synth.GEOM_8B], ids=["d64", "d128"])
@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
def test_decode_per_token_rotation_split_kv(geom, kv):
    """Per-token (mepic) decode through the split-KV kernel: every cached key is
    rotated at its slot position inside the kernel."""
    docs = [[512] * 5, [500, 17, 1023], [16], [700, 700, 3], [33] * 9]
    ks, vs = (0.09, 0.13) if "fp8" in kv else (1.0, 1.0)
    case = synth.build_decode(geom, torch.bfloat16, docs, seed=22, device="cuda", kv_dtype=kv, k_scale=ks,
                              v_scale=vs, variant="mepic")
    got = util.run_cuda(case, "mepic_op", kernel="tensor")
    want = util.run_oracle(case, "mepic_op")
    util.assert_close(got, want, what=f"per-token split-KV decode {kv}", **(FP8 if "fp8" in kv else HALF))


@pytest.mark.parametrize("variant,op", [("lazy", "lazy_op"), ("mepic", "mepic_op")])
@pytest.mark.parametrize("bound", [None, 0, 100, 2000])
def test_decode_covers_sequences_longer_than_max_seq_len(variant, op, bound):
    """``max_seq_len`` only plans the split of the KV range (the reference's decode
    kernel ignores it and walks to ``seq_len``): a bound that is missing, zero or
    smaller than the real lengths must not drop any cached page."""
    docs = [[512] * 9, [500, 17, 1023], [16], [700, 700, 3] * 3, [33] * 9]
    case = synth.build_decode(synth.GEOM_8B, torch.bfloat16, docs, seed=23, device="cuda", kv_dtype="fp8_e4m3",
                              k_scale=0.09, v_scale=0.13, variant=variant)
    want = util.run_oracle(case, op)
    case["max_seq_len"] = bound
    got = util.run_cuda(case, op, kernel="tensor")
    util.assert_close(got, want, what=f"decode with max_seq_len={bound}", **FP8)


@pytest.mark.parametrize("kernel", ["general", "tensor"])
@pytest.mark.parametrize("variant", ["lazy", "mepic"])
def test_prefill_reads_the_packed_table(kernel, variant):
    """One 8-byte packed entry per page instead of three int32 gathers: the result must be
    the same bit for bit, also when the three tables hold garbage the kernel must not read."""
    import lazy_attention_b200 as la
    pool = [100, 64, 33, 250, 16, 129]
    reqs = [dict(docs=[2, 0, 1], qlen=37), dict(docs=[3, 1, 5], qlen=300), dict(docs=[0], qlen=16, lazy=False)]
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, pool, reqs, seed=7, variant=variant, device="cuda")
    packed = util.pack_host(case).to("cuda")
    fn = la.context_attention_fwd if variant == "lazy" else la.context_attention_fwd_mepic

    def run(q_offset, q_mask, packed_table):
        out = util.new_out(case)
        kw = dict(is_lazy=case["is_lazy"]) if variant == "lazy" else {}
        fn(case["q"], case["k"], case["v"], out, "auto", case["k_cache"], case["v_cache"], case["block_table"],
           case["query_start_loc"], case["seq_lens"], case["max_seq_len"], case["max_query_len"],
           case["k_scale"], case["v_scale"], sm_scale=case["sm_scale"], cos_sin_cache=case["cos_sin_cache"],
           q_offset=q_offset, q_mask=q_mask, kernel=kernel, packed_block_table=packed_table, **kw)
        torch.cuda.synchronize()
        return out

    want = run(case["q_offset"], case["q_mask"], None)
    junk = torch.full_like(case["q_offset"], 12345)
    got = run(junk, junk, packed)
    assert torch.equal(got, want)
    op = "lazy_prefill" if variant == "lazy" else "mepic_prefill"
    util.assert_close(got.float().cpu(), util.run_oracle(case, op), what="packed-table prefill", **HALF)


def _new_token_slots(case):
    """slot = page * 16 + in-page index of every new token, from the block table (what the
    engine's slot_mapping holds); one of them is marked as padding (-1)."""
    bt = case["block_table"].cpu()
    qsl = case["query_start_loc"].cpu().tolist()
    seq = case["seq_lens"].cpu().tolist()
    BS = case["geom"].block_size
    slots = []
    for b in range(len(seq)):
        qlen = qsl[b + 1] - qsl[b]
        for n in range(qlen):
            pos = seq[b] - qlen + n
            slots.append(int(bt[b, pos // BS]) * BS + pos % BS)
    return torch.tensor(slots, dtype=torch.int64)


@pytest.mark.parametrize("kernel", ["general", "tensor"])
@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
@pytest.mark.parametrize("variant,op", [("lazy", "lazy_op"), ("mepic", "mepic_op")])
def test_fused_cache_write_equals_separate_write(kernel, kv, variant, op):
    """With ``slot_mapping`` the attention call stores the new K/V rows itself: caches and
    output must equal, bit for bit, a separate write_to_paged_cache followed by the call."""
    import lazy_attention_b200 as la
    reqs = [dict(docs=[2, 0, 1], qlen=37), dict(docs=[3, 1, 5], qlen=300), dict(docs=[1, 2, 4], qlen=1),
            dict(docs=[0], qlen=16, lazy=False), dict(docs=[4, 3], qlen=1), dict(docs=[], qlen=20)]
    ks, vs = (0.11, 0.07) if "fp8" in kv else (1.0, 1.0)
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, POOL, reqs, seed=9, variant=variant, device="cuda",
                               kv_dtype=kv, k_scale=ks, v_scale=vs)
    case["packed_block_table"] = util.pack_host(case).cuda()
    slots = _new_token_slots(case).cuda()
    fn = la.chunked_prefill_paged_decode if variant == "lazy" else la.chunked_prefill_paged_decode_mepic

    def run(kc, vc, slot_mapping):
        out = util.new_out(case)
        kw = dict(is_lazy=case["is_lazy"], packed_block_table=case["packed_block_table"]) if variant == "lazy" else {}
        fn(case["q"], case["k"], case["v"], out, kv, kc, vc, case["block_table"], case["query_start_loc"],
           case["seq_lens"], case["max_seq_len"], case["max_query_len"], case["k_scale"], case["v_scale"],
           sm_scale=case["sm_scale"], cos_sin_cache=case["cos_sin_cache"], q_offset=case["q_offset"],
           q_mask=case["q_mask"], kernel=kernel, slot_mapping=slot_mapping, **kw)
        torch.cuda.synchronize()
        assert la.device_status() == 0
        return out

    # padding tokens (negative slots) are skipped by both ways: a few prefill tokens and one decode row
    slots[5] = -1
    slots[40:44] = -1
    slots[int(case["query_start_loc"][2])] = -1
    kc_a, vc_a = case["k_cache"].clone(), case["v_cache"].clone()
    la.write_to_paged_cache(case["k"], case["v"], kc_a, vc_a, slots, kv, case["k_scale"], case["v_scale"])
    out_a = run(kc_a, vc_a, None)
    kc_b, vc_b = case["k_cache"].clone(), case["v_cache"].clone()
    out_b = run(kc_b, vc_b, slots)
    assert torch.equal(kc_a, kc_b), "K cache differs from the separate write"
    assert torch.equal(vc_a, vc_b), "V cache differs from the separate write"
    assert torch.equal(out_a, out_b), "attention output differs"
    assert not torch.equal(kc_b, case["k_cache"]), "nothing was written"


@pytest.mark.parametrize("geom", [synth.GEOM_1B, synth.GEOM_8B], ids=["d64", "d128"])
@pytest.mark.parametrize("variant,op", [("lazy", "lazy_op"), ("mepic", "mepic_op")])
def test_fused_rotary_op_on_the_query(geom, variant, op):
    """``positions`` makes the kernels apply the query-only rotary op themselves: the result
    must match the oracle run on a query that the op (oracle restatement, rounded to bf16)
    has rotated beforehand, and the query tensor must be left as it was."""
    import lazy_attention_b200 as la
    reqs = [dict(docs=[2, 0, 1], qlen=37), dict(docs=[3, 1, 5], qlen=300), dict(docs=[1, 2, 4], qlen=1),
            dict(docs=[0], qlen=16, lazy=False), dict(docs=[4, 3], qlen=1)]
    case = synth.build_prefill(geom, torch.bfloat16, POOL, reqs, seed=10, variant=variant, device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    g = torch.Generator().manual_seed(1)
    rows = case["cos_sin_cache"].shape[0]
    positions = torch.randint(0, rows, (case["q"].shape[0],), generator=g, dtype=torch.int64)
    positions[3] = 0
    rotated = dict(case)
    rotated["q"] = oracle.apply_rotary_q(case["q"].cpu(), positions, case["cos_sin_cache"].cpu())
    want = util.run_oracle(rotated, op)
    q_before = case["q"].clone()
    out = util.new_out(case)
    fn = la.chunked_prefill_paged_decode if variant == "lazy" else la.chunked_prefill_paged_decode_mepic
    kw = dict(is_lazy=case["is_lazy"], packed_block_table=case["packed_block_table"]) if variant == "lazy" else {}
    fn(case["q"], case["k"], case["v"], out, "auto", case["k_cache"], case["v_cache"], case["block_table"],
       case["query_start_loc"], case["seq_lens"], case["max_seq_len"], case["max_query_len"], case["k_scale"],
       case["v_scale"], sm_scale=case["sm_scale"], cos_sin_cache=case["cos_sin_cache"], q_offset=case["q_offset"],
       q_mask=case["q_mask"], kernel="tensor", positions=positions.cuda(), **kw)
    torch.cuda.synchronize()
    assert la.device_status() == 0
    assert torch.equal(case["q"], q_before), "the query tensor was modified"
    util.assert_close(out.float().cpu(), want, what=f"fused rotary {variant}", **HALF)
    with pytest.raises(NotImplementedError, match="rotary"):
        fn(case["q"], case["k"], case["v"], out, "auto", case["k_cache"], case["v_cache"], case["block_table"],
           case["query_start_loc"], case["seq_lens"], case["max_seq_len"], case["max_query_len"], case["k_scale"],
           case["v_scale"], sm_scale=case["sm_scale"], cos_sin_cache=case["cos_sin_cache"],
           q_offset=case["q_offset"], q_mask=case["q_mask"], kernel="general", positions=positions.cuda(), **kw)


@pytest.mark.parametrize("geom", [synth.GEOM_1B, synth.GEOM_8B], ids=["d64", "d128"])
@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
@pytest.mark.parametrize("llama3", [True, False], ids=["llama3", "plain"])
def test_decode_computes_cos_sin_in_the_kernel(geom, kv, llama3, monkeypatch):
    """LAZY_DECODE_COMPUTE_COS_SIN=1: the decode kernel takes cos/sin(position * inv_freq) from
    the rotary layer's parameters instead of a table row.  Checked against the oracle with an
    unrounded float32 table, and against the table path within the reference's own bound for
    this switch (0.02 absolute, benchmarks/bench_rope_cos_sin.py:133)."""
    import lazy_attention_b200 as la
    docs = [[512] * 5, [500, 17, 1023], [16], [700, 700, 3], [33] * 9]
    ks, vs = (0.09, 0.13) if "fp8" in kv else (1.0, 1.0)
    case = synth.build_decode(geom, torch.bfloat16, docs, seed=24, device="cuda", kv_dtype=kv, k_scale=ks,
                              v_scale=vs, llama3=llama3)
    meta = dict(ROPE_TYPE=1 if llama3 else 0, BASE=geom.rope_theta, ORIG_MAX_POSITION=8192,
                SCALING_FACTOR=8.0 if llama3 else 1.0, LOW_FACTOR=1.0, HIGH_FACTOR=4.0 if llama3 else 1.0)
    table_out = util.run_cuda(case, "lazy_op", kernel="tensor")
    exact = dict(case)
    exact["cos_sin_cache"] = oracle.build_cos_sin_table(case["cos_sin_cache"].shape[0], geom.head_dim, geom.rope_theta,
                                                        oracle.ROPE_LLAMA3 if llama3 else oracle.ROPE_DEFAULT,
                                                        **(synth.LLAMA3_SCALING if llama3 else {}))
    want = util.run_oracle(exact, "lazy_op")
    monkeypatch.setenv("LAZY_DECODE_COMPUTE_COS_SIN", "1")
    out = util.new_out(case)
    la.chunked_prefill_paged_decode(case["q"], case["k"], case["v"], out, kv, case["k_cache"], case["v_cache"],
                                    case["block_table"], case["query_start_loc"], case["seq_lens"],
                                    case["max_seq_len"], 1, case["k_scale"], case["v_scale"],
                                    sm_scale=case["sm_scale"], cos_sin_cache=None, rope_meta=meta,
                                    is_lazy=case["is_lazy"], q_offset=case["q_offset"], q_mask=case["q_mask"],
                                    packed_block_table=case["packed_block_table"], kernel="tensor")
    torch.cuda.synchronize()
    assert la.device_status() == 0
    got = out.float().cpu()
    util.assert_close(got, want, what="in-kernel cos/sin vs oracle", **(FP8 if "fp8" in kv else HALF))
    assert float((got - table_out).abs().max()) < 0.02, "computed and loaded cos/sin disagree"


def test_empty_batch_and_skip_decode_leave_output_untouched():
    import lazy_attention_b200 as la
    case = util.to_device(util.load_golden("lazy_prefill_small"), "cuda")
    out = torch.full_like(util.new_out(case), 7.0)
    la.context_attention_fwd(case["q"], case["k"], case["v"], out, "auto", case["k_cache"], case["v_cache"],
                             case["block_table"], case["query_start_loc"], case["seq_lens"],
                             case["max_seq_len"], case["max_query_len"], case["k_scale"], case["v_scale"],
                             sm_scale=case["sm_scale"], skip_decode=True, cos_sin_cache=case["cos_sin_cache"],
                             rotary_dim=32, is_lazy=case["is_lazy"], q_offset=case["q_offset"],
                             q_mask=case["q_mask"], kernel="general")
    torch.cuda.synchronize()
    start = case["query_start_loc"].cpu()
    for b in range(len(start) - 1):
        rows = out[int(start[b]):int(start[b + 1])]
        if int(start[b + 1]) - int(start[b]) == 1:
            assert bool((rows == 7.0).all()), "decode row was written by the prefill kernel"
        else:
            assert bool((rows != 7.0).any())
    empty = torch.zeros(0, dtype=torch.int32, device="cuda")
    la.context_attention_fwd(case["q"][:0], case["k"][:0], case["v"][:0], out[:0], "auto", case["k_cache"],
                             case["v_cache"], case["block_table"][:0], torch.zeros(1, dtype=torch.int32, device="cuda"),
                             empty, 0, 0, case["k_scale"], case["v_scale"])


@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3", "fp8_e5m2"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "fp16", "fp32"])
def test_write_to_paged_cache_bit_exact(kv, dtype):
    """New K/V rows land in the page / in-page slot the mapping names, bit for bit
    (fp8: the same saturating conversion of x / scale as torch's)."""
    import lazy_attention_b200 as la
    g = torch.Generator().manual_seed(3)
    Hkv, D, BS, nb, T = 4, 64, 16, 9, 37
    store = torch.uint8 if "fp8" in kv else dtype
    x = 16 if "fp8" in kv else 16 // torch.empty((), dtype=dtype).element_size()
    kc = torch.zeros((nb, Hkv, D // x, BS, x), dtype=store)
    vc = torch.zeros((nb, Hkv, D, BS), dtype=store)
    key = (torch.randn((T, Hkv, D), generator=g) * 3).to(dtype)
    val = (torch.randn((T, Hkv, D), generator=g) * 300).to(dtype)  # large: exercises fp8 saturation
    slots = torch.randperm(nb * BS, generator=g)[:T].to(torch.int64)
    slots[5] = -1
    ks, vs = torch.tensor([0.07]), torch.tensor([0.21])
    kc_ref, vc_ref = kc.clone(), vc.clone()
    oracle.write_to_paged_cache(key, val, kc_ref, vc_ref, slots, kv, ks, vs)
    kc_d, vc_d = kc.cuda(), vc.cuda()
    la.write_to_paged_cache(key.cuda(), val.cuda(), kc_d, vc_d, slots.cuda(), kv, ks.cuda(), vs.cuda())
    torch.cuda.synchronize()
    assert torch.equal(kc_d.cpu().view(torch.uint8), kc_ref.view(torch.uint8))
    assert torch.equal(vc_d.cpu().view(torch.uint8), vc_ref.view(torch.uint8))


# ---- integer path on the GPU -------------------------------------------------------------
def test_pack_block_table_bit_exact():
    import lazy_attention_b200 as la
    rng = np.random.default_rng(0)
    bt = rng.integers(0, 2**31 - 1, size=(37, 513), dtype=np.int64).astype(np.int32)
    off = rng.integers(0, 0x10000, size=bt.shape).astype(np.int32)
    msk = rng.integers(0, 16, size=bt.shape).astype(np.int32)
    want = oracle.pack_block_table(bt, off, msk)
    got = la.pack_block_table(torch.from_numpy(bt).cuda(), torch.from_numpy(off).cuda(),
                              torch.from_numpy(msk).cuda())
    assert np.array_equal(got.cpu().numpy(), want)
    # overflow carries into the block id exactly as int64 arithmetic does
    off[0, 0] = 0x10000
    bt[0, 0] = 6
    got = la.pack_block_table(torch.from_numpy(bt).cuda(), torch.from_numpy(off).cuda(),
                              torch.from_numpy(msk).cuda())
    assert int(got[0, 0].item() >> 32) == 7
    # row-wise rebuild touches only the listed rows
    out = torch.full((37, 513), -1, dtype=torch.int64, device="cuda")
    rows = torch.tensor([3, 36, 10], dtype=torch.int32, device="cuda")
    la.pack_block_table(torch.from_numpy(bt).cuda(), torch.from_numpy(off).cuda(),
                        torch.from_numpy(msk).cuda(), out=out, rows=rows)
    want = oracle.pack_block_table(bt, off, msk)
    o = out.cpu().numpy()
    for r in range(37):
        if r in (3, 36, 10):
            assert np.array_equal(o[r], want[r])
        else:
            assert (o[r] == -1).all()


def test_metadata_buffers_pack_per_group():
    import lazy_attention_b200 as la
    from types import SimpleNamespace
    buf = la.LazyMetadataBuffers(4, 6, device="cuda", num_kv_groups=2)
    reqs = [SimpleNamespace(is_lazy=True, lazy_variant=1, q_offset=[5, 5, 1], q_mask=[0, 3, 0]),
            SimpleNamespace(is_lazy=False, lazy_variant=0, q_offset=None, q_mask=None)]
    buf.refresh(reqs)
    t0 = torch.arange(24, dtype=torch.int32, device="cuda").reshape(4, 6)
    t1 = t0 + 100
    assert buf.rebuild_packed_block_table([t0, t1], 2) == 2
    for g, t in enumerate((t0, t1)):
        want = oracle.pack_block_table(t.cpu().numpy()[:2], buf.lazy_offset_cpu.numpy()[:2],
                                       buf.lazy_mask_cpu.numpy()[:2])
        assert np.array_equal(buf.packed_block_tables[g][:2].cpu().numpy(), want)
    assert buf.rebuild_packed_block_table([t0, t1], 2) == 0
    t0[1, 2] = 77
    buf.mark_rows_changed([1])
    assert buf.rebuild_packed_block_table([t0, t1], 2) == 1
    assert int(buf.packed_block_tables[0][1, 2].item() >> 32) == 77
    md = buf.attach(SimpleNamespace(), 2, group_idx=1)
    assert md.packed_block_table.shape == (2, 6) and md.is_lazy.tolist() == [True, False]


@pytest.mark.parametrize("llama3", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cos_sin_table(llama3, dtype):
    import lazy_attention_b200 as la
    kw = dict(scaling_factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, orig_max_position=8192)
    rope_type = la.ROPE_LLAMA3 if llama3 else la.ROPE_DEFAULT
    got = la.build_cos_sin_table(70000, 128, 500000.0, rope_type, dtype=dtype, **kw).float().cpu()
    want = oracle.build_cos_sin_table(70000, 128, 500000.0, rope_type, **kw)
    # float32 angles: one ulp of the frequency times the position
    pos = torch.arange(70000, dtype=torch.float32)[:, None]
    bound = 2e-6 + pos * 2.4e-7 + (4e-3 if dtype == torch.bfloat16 else 0.0)
    assert bool(((got - want).abs() <= bound).all())
    assert torch.equal(got[0, :64], torch.ones(64)) and torch.equal(got[0, 64:], torch.zeros(64))


@pytest.mark.parametrize("variant,op", [("lazy", "lazy_op")])
@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
def test_rotation_offsets_at_the_16_bit_limit(variant, op, kv):
    """Pages whose rotation offset is the largest the packed table can carry (65535, i.e. row
    65534 of the cos/sin table), in a prefill request and in a decode row: the offset must
    survive the 16-bit field of the packed entry and reach the table lookup intact."""
    import lazy_attention_b200 as la
    reqs = [dict(docs=[2, 0, 1], qlen=130), dict(docs=[3, 1], qlen=1), dict(docs=[5, 4], qlen=40)]
    ks, vs = (0.11, 0.07) if "fp8" in kv else (1.0, 1.0)
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, POOL, reqs, seed=17, variant=variant, device="cuda",
                               kv_dtype=kv, k_scale=ks, v_scale=vs, max_position=la.MAX_PACKED_Q_OFFSET + 1)
    assert case["cos_sin_cache"].shape[0] == la.MAX_PACKED_Q_OFFSET + 1
    off = case["q_offset"]
    for b in range(off.shape[0]):
        rows = torch.nonzero(off[b] > 1).flatten()
        assert rows.numel() > 0
        off[b, rows[-1]] = la.MAX_PACKED_Q_OFFSET          # the last rotating page of the request
        off[b, rows[0]] = la.MAX_PACKED_Q_OFFSET - 1
        off[b, rows[rows.numel() // 2]] = 32768             # the first value with the field's top bit set
    case["packed_block_table"] = util.pack_host(case).cuda()
    want = util.run_oracle(case, op)
    for kernel in ("tensor", "general"):
        got = util.run_cuda(case, op, kernel=kernel)
        util.assert_close(got, want, what=f"offsets at the limit, {kv}, {kernel}", **(FP8 if "fp8" in kv else HALF))
