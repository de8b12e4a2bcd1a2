"""The allocation-free prefill entry point against the regular one.

Some users of this library may not allocate device memory around the attention
call -- all free HBM already belongs to the KV cache, or the call sits where
cudaMalloc's device-wide synchronisation is not acceptable -- so they cannot
supply the split-KV scratch.  ``la_prefill_fwd_noalloc`` keeps that scratch in a
fixed 32 MiB array inside the library.  This test drives it through the C ABI on
a call that really splits the KV range, twice in a row (the array keeps the
first call's contents), and checks both results against ``la_prefill_fwd`` and
against the CPU oracle within the tolerance the other bf16 tests use.  It also checks that a call too
large for the array is refused with a message that names both sizes.

The file sorts last on purpose: with ``pytest -x`` every other test has run
before this one.
"""
import pytest
import torch

import util
from lazy_attention_b200 import synth
from lazy_attention_b200.no_alloc import context_attention_fwd_no_alloc

pytestmark = pytest.mark.gpu

HALF = dict(atol=2e-2, rtol=1e-2)


def _call_no_alloc(case, out):
    context_attention_fwd_no_alloc(case["q"], case["k"], case["v"], out, case["k_cache"], case["v_cache"],
                                   case["block_table"], case["query_start_loc"], case["seq_lens"],
                                   case["max_seq_len"], case["max_query_len"],
                                   cos_sin_cache=case["cos_sin_cache"], is_lazy=case["is_lazy"],
                                   q_offset=case["q_offset"], q_mask=case["q_mask"],
                                   sm_scale=case["sm_scale"])
    torch.cuda.synchronize()


def test_no_alloc_entry_matches_regular_entry_twice():
    import lazy_attention_b200 as la
    # 1B geometry, one request, 5120 cached tokens, 128 new: few row blocks, so the
    # kernel splits the KV range and goes through the scratch.
    case = synth.config_c2(device="cuda")
    want = util.run_cuda(case, "lazy_prefill", kernel="tensor")
    truth = util.run_oracle(case, "lazy_prefill")
    for attempt in range(2):
        out = torch.full((case["num_tokens"], 32, 64), float("nan"), dtype=torch.bfloat16, device="cuda")
        held = torch.cuda.memory_allocated()
        _call_no_alloc(case, out)
        assert torch.cuda.memory_allocated() == held, "the entry point went through torch's allocator"
        assert la.device_status() == 0
        util.assert_close(out.float().cpu(), want, what=f"no-alloc call {attempt}", **HALF)
        util.assert_close(out.float().cpu(), truth, what=f"no-alloc call {attempt} vs oracle", **HALF)
    # a different call in between must not disturb the next one
    other = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, [512] * 4, [dict(docs=[3, 1, 0, 2], qlen=64)],
                                seed=5, device="cuda")
    out2 = util.new_out(other)
    _call_no_alloc(other, out2)
    util.assert_close(out2.float().cpu(), util.run_cuda(other, "lazy_prefill", kernel="tensor"),
                      what="no-alloc, second shape", **HALF)
    out3 = util.new_out(case)
    _call_no_alloc(case, out3)
    util.assert_close(out3.float().cpu(), want, what="no-alloc after another shape", **HALF)


def test_no_alloc_entry_refuses_what_does_not_fit(monkeypatch):
    from lazy_attention_b200 import no_alloc
    # Five requests of that shape, with the split count pinned to 8 (the library's tuning
    # switch; the planner itself would not split a batch this wide): 43 MB of partials.
    monkeypatch.setenv("LAZY_ATTN_B200_PREFILL_SPLITS", "8")
    pool = [512] * 50
    reqs = [dict(docs=list(range(10 * b, 10 * b + 10)), qlen=128) for b in range(5)]
    case = synth.build_prefill(synth.GEOM_1B, torch.bfloat16, pool, reqs, seed=2, device="cuda")
    out = util.new_out(case)
    args = (case["q"], case["k"], case["v"], out, case["k_cache"], case["v_cache"], case["block_table"],
            case["query_start_loc"], case["seq_lens"], case["max_seq_len"], case["max_query_len"])
    assert no_alloc.scratch_need(*args) > no_alloc.NO_ALLOC_SCRATCH_BYTES, "pick a larger case"
    with pytest.raises(RuntimeError, match="built-in scratch holds"):
        _call_no_alloc(case, out)
    # shapes outside the tensor-core kernel are refused, not silently rerouted
    small = synth.build_prefill(synth.Geometry(4, 2, 32, 16), torch.float16, [64], [dict(docs=[0], qlen=8)],
                                seed=2, device="cuda")
    with pytest.raises(NotImplementedError, match="head_dim"):
        _call_no_alloc(small, util.new_out(small))
