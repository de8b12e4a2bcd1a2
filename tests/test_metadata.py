"""Host-side integer path of the library (scheduler metadata, offset bound,
request buffers) -- bit-exact against the reference's vectors.  CPU only."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import lazy_attention_b200 as la
import util
from oracle import lazy_oracle as oracle


def test_reference_unit_test_vector():
    req = SimpleNamespace(document_lens=[6, 15, 8, 2], document_lens_padded=[8, 16, 8, 8])
    q_offset, q_mask = la.metadata_for_lazy_attention(req, 8)
    assert q_offset == [10, 16, 16, 31, 39, 1]
    assert q_mask == [2, 0, 1, 0, 6, 0]
    q_offset2, q_mask2 = la.metadata_for_mepic(req, 8)
    assert q_offset2 == [0] * len(q_offset) and q_mask2 == q_mask


def test_vectors_from_reference_function():
    for c in util.metadata_vectors()["cases"]:
        off, msk = la.metadata_for_lazy_attention(c["lens"], c["padded"], c["bs"])
        assert off == c["q_offset"] and msk == c["q_mask"]
        assert la.max_rotation_offset(c["lens"], c["padded"]) == c["max_rot"]
        assert (off, msk) == oracle.metadata_for_lazy_attention(c["lens"], c["padded"], c["bs"])


@pytest.mark.parametrize("lens", [[6], [16, 16], [6, 15, 8, 2], [1, 1, 1, 1, 1], [4096, 17], [100] * 32])
def test_bound_helper_agrees_with_metadata(lens):
    padded = [(n + 15) // 16 * 16 for n in lens]
    off, _ = la.metadata_for_lazy_attention(lens, padded, 16)
    assert la.max_rotation_offset(lens, padded) == max(off)


def test_offset_bound_cases():
    huge = la.MAX_PACKED_Q_OFFSET * 4
    assert la.max_rotation_offset([huge], [huge]) == 1
    la.validate_rotation_offsets([huge], [huge])
    assert la.max_rotation_offset([1024] * 64, [1024] * 64) == 1024 * 63 + 1
    la.validate_rotation_offsets([1024] * 64, [1024] * 64)
    with pytest.raises(ValueError, match="past the"):
        la.validate_rotation_offsets([1024] * 65, [1024] * 65)
    assert la.max_rotation_offset([1] * 8, [16] * 8) == 8 * 15 + 7 + 1
    assert la.max_rotation_offset([], []) == 0


def test_variant_switch(monkeypatch):
    req = SimpleNamespace(document_lens=[5, 16], document_lens_padded=[16, 16])
    monkeypatch.delenv("LAZY_ATTENTION_VARIANT", raising=False)
    assert la.metadata_for_variant(req, 16)[0] == [12, 17, 1]
    monkeypatch.setenv("LAZY_ATTENTION_VARIANT", "mepic")
    assert la.metadata_for_variant(req, 16)[0] == [0, 0, 0]


def _req(q_offset, lazy=True):
    return SimpleNamespace(is_lazy=lazy, lazy_variant=1, q_offset=q_offset,
                           q_mask=[0] * len(q_offset), req_id="req-0")


def test_buffers_accept_limit_and_refuse_overflow():
    buf = la.LazyMetadataBuffers(2, 8, device="cpu", pin_memory=False)
    buf.refresh([_req([1, la.MAX_PACKED_Q_OFFSET])])
    assert int(buf.lazy_offset_np[0, 1]) == la.MAX_PACKED_Q_OFFSET
    assert bool(buf.is_lazy_req[0]) and int(buf.lazy_offset[0, 1]) == la.MAX_PACKED_Q_OFFSET
    with pytest.raises(ValueError, match="does not fit the 16 bits"):
        buf.refresh([_req([1, la.MAX_PACKED_Q_OFFSET + 1])])


def test_buffers_zero_rows_of_plain_requests():
    buf = la.LazyMetadataBuffers(3, 4, device="cpu", pin_memory=False)
    buf.refresh([_req([7, 7, 1]), _req([9], lazy=False)])
    assert buf.lazy_offset_cpu[0].tolist() == [7, 7, 1, 0]
    assert buf.lazy_offset_cpu[1].tolist() == [0, 0, 0, 0]
    assert buf.is_lazy_req_cpu.tolist() == [True, False, False]
    buf.refresh([_req([3], lazy=False)])
    assert buf.lazy_offset_cpu[0].tolist() == [0, 0, 0, 0]


def test_pack_refuses_cpu_tensors():
    z = torch.zeros((1, 4), dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        la.pack_block_table(z, z, z)


def test_ops_refuse_cpu_tensors():
    case = util.load_golden("lazy_prefill_small")
    out = util.new_out(case)
    with pytest.raises(RuntimeError, match="CUDA"):
        la.context_attention_fwd(case["q"], case["k"], case["v"], out, "auto", case["k_cache"],
                                 case["v_cache"], case["block_table"], case["query_start_loc"],
                                 case["seq_lens"], case["max_seq_len"], case["max_query_len"],
                                 case["k_scale"], case["v_scale"], cos_sin_cache=case["cos_sin_cache"],
                                 rotary_dim=32, is_lazy=case["is_lazy"], q_offset=case["q_offset"],
                                 q_mask=case["q_mask"])


def test_argument_errors_match_reference():
    case = util.load_golden("lazy_prefill_small")
    out = util.new_out(case)
    args = (case["q"], case["k"], case["v"], out)
    rest = (case["block_table"], case["query_start_loc"], case["seq_lens"], case["max_seq_len"],
            case["max_query_len"], case["k_scale"], case["v_scale"])
    u8k = torch.zeros(case["k_cache"].shape, dtype=torch.uint8)
    u8v = torch.zeros(case["v_cache"].shape, dtype=torch.uint8)
    with pytest.raises(ValueError, match="Unsupported FP8"):
        la.context_attention_fwd(*args, "fp8_e3m4", u8k, u8v, *rest)
    with pytest.raises(ValueError, match="auto"):
        la.context_attention_fwd(*args, "auto", u8k, u8v, *rest)
    with pytest.raises(AssertionError):
        la.context_attention_fwd(*args, "fp8", case["k_cache"], case["v_cache"], *rest)
    with pytest.raises(NotImplementedError, match="Alibi"):
        la.context_attention_fwd(*args, "auto", case["k_cache"], case["v_cache"], *rest,
                                 alibi_slopes=torch.ones(4))


def test_metadata_properties_hold_for_random_document_sets():
    """Properties the kernels rely on, over random document sets (hypothesis): one entry per
    page plus the query page; the largest offset is what max_rotation_offset announces; offsets
    never decrease from one document to the next; every pad count is below a page and sits on
    its document's last page; the per-token variant has the same pads and no offsets."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=200, deadline=None)
    @given(st.lists(st.integers(min_value=1, max_value=3000), min_size=0, max_size=12),
           st.sampled_from([16, 32]))
    def check(lens, bs):
        padded = [(n + bs - 1) // bs * bs for n in lens]
        off, msk = la.metadata_for_lazy_attention(lens, padded, bs)
        pages = sum(padded) // bs
        assert len(off) == len(msk) == pages + 1
        assert off[-1] == 1 and msk[-1] == 0
        if lens:
            assert max(off[:-1]) == la.max_rotation_offset(lens, padded)
            assert all(a <= b for a, b in zip(off[:-2], off[1:-1]))
        cursor = 0
        for n, p in zip(lens, padded):
            k = p // bs
            assert len(set(off[cursor:cursor + k])) == 1, "one offset per document"
            assert all(m == 0 for m in msk[cursor:cursor + k - 1])
            assert msk[cursor + k - 1] == p - n and 0 <= p - n < bs
            cursor += k
        off_m, msk_m = la.metadata_for_mepic(lens, padded, bs)
        assert msk_m == msk and not any(off_m)
        if lens and la.max_rotation_offset(lens, padded) > la.MAX_PACKED_Q_OFFSET:
            with pytest.raises(ValueError):
                la.validate_rotation_offsets(lens, padded)
        else:
            la.validate_rotation_offsets(lens, padded)

    check()
