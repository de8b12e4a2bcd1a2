"""The oracle against what the reference itself computes.

Floating point: fixtures under tests/golden/ hold inputs and the outputs of the
reference's Triton kernels run through Triton's CPU interpreter in float32
(tests/golden/make_golden.py).  Integer: the golden vectors of the reference's
own unit tests plus vectors produced by its scheduler function.
"""
import numpy as np
import pytest
import torch

import util
from lazy_attention_b200 import synth
from oracle import lazy_oracle as oracle

TOL = dict(atol=2e-5, rtol=1e-5)

FLOAT_CASES = [
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


@pytest.mark.parametrize("name,op,kw", FLOAT_CASES, ids=[c[0] for c in FLOAT_CASES])
def test_oracle_matches_reference_kernels(name, op, kw):
    case = util.load_golden(name)
    got = util.run_oracle(case, op, **kw)
    util.assert_close(got, case["out"], what=name, **TOL)


@pytest.mark.parametrize("variant", ["lazy", "mepic"])
def test_oracle_matches_reference_on_first_config(variant):
    """BASELINE config 1: 1B geometry, fp32, batch 2, 3x128-token documents at
    seeded random slots, 32 new tokens.  The fixture keeps four heads of the
    reference kernel's output; the inputs are rebuilt from the seed and checked
    by checksum."""
    z = np.load(util.GOLDEN / f"c1_{variant}.npz")
    case = synth.config_c1(variant=variant)
    assert abs(case["q"].double().sum().item() - float(z["q_checksum"])) < 1e-6
    assert abs(case["k_cache"].double().sum().item() - float(z["kc_checksum"])) < 1e-6
    case["packed_block_table"] = util.pack_host(case)
    op = "lazy_prefill" if variant == "lazy" else "mepic_op"
    got = util.run_oracle(case, op)
    want = torch.from_numpy(z["out_heads"])
    heads = [int(h) for h in z["heads"]]
    util.assert_close(got[:, heads], want, atol=1e-5, rtol=1e-5, what=f"c1 {variant}")


# ---- integer path -------------------------------------------------------------------
def test_scheduler_golden_vector():
    # lazy_attn/tests/core/test_scheduler.py:36-61
    off, msk = oracle.metadata_for_lazy_attention([6, 15, 8, 2], [8, 16, 8, 8], 8)
    assert off == [10, 16, 16, 31, 39, 1]
    assert msk == [2, 0, 1, 0, 6, 0]
    off2, msk2 = oracle.metadata_for_mepic([6, 15, 8, 2], [8, 16, 8, 8], 8)
    assert off2 == [0] * 6 and msk2 == msk


def test_metadata_vectors_from_reference_function():
    vec = util.metadata_vectors()
    assert vec["max_packed_q_offset"] == oracle.MAX_PACKED_Q_OFFSET == 0xFFFF
    for c in vec["cases"]:
        off, msk = oracle.metadata_for_lazy_attention(c["lens"], c["padded"], c["bs"])
        assert off == c["q_offset"] and msk == c["q_mask"], c["lens"]
        assert oracle.max_rotation_offset(c["lens"], c["padded"]) == c["max_rot"]
        if c["lens"]:
            assert max(off) == c["max_rot"]


def test_rotation_offset_bounds():
    # lazy_attn/tests/core/test_rotation_offset_bound.py:19-75
    huge = 0xFFFF * 4
    assert oracle.max_rotation_offset([huge], [huge]) == 1
    assert oracle.max_rotation_offset([1024] * 64, [1024] * 64) == 1024 * 63 + 1
    assert oracle.max_rotation_offset([1024] * 65, [1024] * 65) > 0xFFFF
    assert oracle.max_rotation_offset([1] * 8, [16] * 8) == 8 * 15 + 7 + 1


def test_pack_limit_and_overflow_arithmetic():
    # lazy_attn/tests/worker/test_q_offset_range.py:54-79
    packed = oracle.pack_block_table(np.array([[6]]), np.array([[0x10000]]), np.array([[0]]))
    assert int((packed[0, 0] >> 32) & 0xFFFFFFFF) == 7
    assert int((packed[0, 0] >> 16) & 0xFFFF) == 0
    packed = oracle.pack_block_table(np.array([[6]]), np.array([[0xFFFF]]), np.array([[3]]))
    blk, rot, pad = oracle.unpack_block_table(packed)
    assert (int(blk[0, 0]), int(rot[0, 0]), int(pad[0, 0])) == (6, 0xFFFF, 3)


def test_cos_sin_table_layout_and_llama3_mirror():
    # row pos = [cos | sin]; llama3 smoothing as lazy/model_executor/rope/cos_sin.py:127-148
    tab = oracle.build_cos_sin_table(64, 32, 500000.0, oracle.ROPE_LLAMA3, 8.0, 1.0, 4.0, 8192)
    assert tab.shape == (64, 32)
    assert torch.allclose(tab[0, :16], torch.ones(16)) and torch.allclose(tab[0, 16:], torch.zeros(16))
    assert torch.allclose(tab[:, :16] ** 2 + tab[:, 16:] ** 2, torch.ones(64, 16), atol=1e-6)
    plain = oracle.build_cos_sin_table(64, 32, 500000.0)
    inv = 1.0 / (500000.0 ** (torch.arange(0, 32, 2).float() / 32))
    assert torch.allclose(plain[5, :16], torch.cos(5 * inv))
    # high-frequency dims are untouched by the llama3 scaling, the lowest are divided by 8
    f3 = oracle.rope_inv_freq(128, 500000.0, oracle.ROPE_LLAMA3, 8.0, 1.0, 4.0, 8192)
    f0 = oracle.rope_inv_freq(128, 500000.0)
    assert torch.equal(f3[:8], f0[:8])
    assert torch.allclose(f3[-1], f0[-1] / 8.0)
    assert torch.equal(synth._cos_sin_host(64, 32, 500000.0, True), tab)


def test_slice_case_matches_whole_case():
    """A (request, KV head) slice run through the oracle equals the same rows of
    the whole case (the full-size GPU tests check slices only)."""
    import torch
    from lazy_attention_b200 import synth
    pool = [100, 64, 33, 250, 16, 129]
    reqs = [dict(docs=[2, 0, 1], qlen=37), dict(docs=[3, 1, 5], qlen=20), dict(docs=[4], qlen=1)]
    for variant, op in (("lazy", "lazy_op"), ("mepic", "mepic_op")):
        case = synth.build_prefill(synth.GEOM_1B, torch.float32, pool, reqs, seed=11, variant=variant)
        case["packed_block_table"] = util.pack_host(case)
        whole = util.run_oracle(case, op)
        for b, h in ((0, 0), (1, 5), (2, 7)):
            sub = util.slice_case(case, b, h)
            (s0, s1), (h0, h1) = sub["token_range"], sub["head_range"]
            got = util.run_oracle(sub, op)
            assert float((got - whole[s0:s1, h0:h1]).abs().max()) < 1e-5


def test_cos_sin_table_matches_reference_mirror():
    """The oracle's llama3 table against rows of the reference's own torch mirror
    (lazy_attn/lazy/model_executor/rope/cos_sin.py:127-148), stored by make_golden.py."""
    z = np.load(util.GOLDEN / "cos_sin_llama3.npz")
    base, factor, low, high, orig = (float(v) for v in z["params"])
    positions = [int(v) for v in z["positions"]]
    for head in (64, 128):
        table = oracle.build_cos_sin_table(max(positions) + 1, head, base, oracle.ROPE_LLAMA3, factor, low, high,
                                           int(orig))
        rows = table[positions]
        half = head // 2
        # the mirror returns the NeoX-duplicated layout [head]; the table keeps one half each
        want_cos, want_sin = torch.from_numpy(z[f"cos_{head}"]), torch.from_numpy(z[f"sin_{head}"])
        assert torch.equal(want_cos[:, :half], want_cos[:, half:])
        # float32 evaluation order differs slightly (theta = pos * inv): a few ulp of the angle
        assert float((rows[:, :half] - want_cos[:, :half]).abs().max()) < 2e-3
        assert float((rows[:, half:] - want_sin[:, :half]).abs().max()) < 2e-3
        small = [i for i, pos in enumerate(positions) if pos <= 4097]
        assert float((rows[small][:, :half] - want_cos[small][:, :half]).abs().max()) < 1e-6
        assert float((rows[small][:, half:] - want_sin[small][:, :half]).abs().max()) < 1e-6
