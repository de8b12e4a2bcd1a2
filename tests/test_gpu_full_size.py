"""BASELINE configurations c3, c4 and c5 at their full sizes on the GPU.

The float32 oracle cannot run a whole call of these sizes in seconds, so each
test checks
  * slices: single (request, KV head) pairs cut out of the full case and run
    through the oracle at the full context length (`util.slice_case`),
  * the whole output against the general SIMT kernel (an independent
    implementation that the small cases pin to the oracle),
  * size-independent properties: bit-identical results on a second run and
    under a permutation of the physical pages, and rows of probabilities that
    sum to one (a value cache of ones must give ones).
Tolerances: bf16 max-abs 2e-2 / rel 1e-2; fp8 caches 5e-2 abs.
"""
import pytest
import torch

import util
from lazy_attention_b200 import synth

pytestmark = pytest.mark.gpu

HALF = dict(atol=2e-2, rtol=1e-2)
FP8 = dict(atol=5e-2, rtol=1e-2)


def _check_slices(case, got, op, picks, tol):
    for b, h in picks:
        sub = util.slice_case(case, b, h)
        want = util.run_oracle(sub, op)
        (s0, s1), (h0, h1) = sub["token_range"], sub["head_range"]
        util.assert_close(got[s0:s1, h0:h1], want, what=f"oracle slice request {b} kv head {h}", **tol)


def _prefill_op(variant):
    return "lazy_prefill" if variant == "lazy" else "mepic_prefill"


@pytest.mark.parametrize("variant", ["lazy", "mepic"])
def test_c4_full_size(variant):
    """8 requests x (65536 cached + 512 new tokens), 8B geometry, bf16."""
    case = synth.config_c4(device="cuda", variant=variant)
    op = _prefill_op(variant)
    got = util.run_cuda(case, op, kernel="tensor")
    _check_slices(case, got, op, [(0, 0), (5, 7)], HALF)
    assert torch.equal(got, util.run_cuda(case, op, kernel="tensor")), "second run differs"
    util.assert_close(got, util.run_cuda(case, op, kernel="general"), what="tensor-core vs general kernel", **HALF)
    # probabilities sum to one: values of ones give ones
    case["v_cache"].fill_(1.0)
    case["v"].fill_(1.0)
    ones = util.run_cuda(case, op, kernel="tensor")
    assert float((ones - 1.0).abs().max()) < 1e-2


@pytest.mark.parametrize("variant", ["lazy", "mepic"])
def test_c3_full_size(variant):
    """32 requests x 20 documents of 256..1024 tokens with Zipf reuse, 64..256 new tokens."""
    case = synth.config_c3(device="cuda", variant=variant)
    op = _prefill_op(variant)
    got = util.run_cuda(case, op, kernel="tensor")
    _check_slices(case, got, op, [(0, 1), (17, 4), (31, 6)], HALF)
    util.assert_close(got, util.run_cuda(case, op, kernel="general"), what="tensor-core vs general kernel", **HALF)
    # a permutation of the physical pages changes nothing, bit for bit
    nb = case["k_cache"].shape[0]
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(5)).cuda()
    moved = dict(case)
    for name in ("k_cache", "v_cache"):
        t = torch.empty_like(case[name])
        t[perm] = case[name]
        moved[name] = t
    moved["block_table"] = perm[case["block_table"].long().clamp(0, nb - 1)].to(torch.int32)
    assert torch.equal(got, util.run_cuda(moved, op, kernel="tensor")), "page permutation changed the result"


def test_c5_full_size():
    """256 decode sequences of 4k..16k cached tokens, e4m3 cache, bf16 query."""
    case = synth.config_c5(device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    got = util.run_cuda(case, "lazy_op", kernel="tensor")
    _check_slices(case, got, "lazy_op", [(0, 0), (100, 5), (255, 7)], FP8)
    assert torch.equal(got, util.run_cuda(case, "lazy_op", kernel="tensor")), "second run differs"
    util.assert_close(got, util.run_cuda(case, "lazy_op", kernel="general"), what="split-KV vs general kernel", **FP8)
    # a permutation of the physical pages changes nothing, bit for bit
    nb = case["k_cache"].shape[0]
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(6)).cuda()
    moved = dict(case)
    for name in ("k_cache", "v_cache"):
        t = torch.empty_like(case[name])
        t[perm] = case[name]
        moved[name] = t
    moved["block_table"] = perm[case["block_table"].long().clamp(0, nb - 1)].to(torch.int32)
    moved["packed_block_table"] = util.pack_host(moved).cuda()
    assert torch.equal(got, util.run_cuda(moved, "lazy_op", kernel="tensor")), "page permutation changed the result"
    # probabilities sum to one: a value cache of ones (0x38 in e4m3) gives v_scale
    case["v_cache"].view(torch.uint8).fill_(0x38)
    ones = util.run_cuda(case, "lazy_op", kernel="tensor")
    vs = float(case["v_scale"].reshape(-1)[0])
    assert float((ones / vs - 1.0).abs().max()) < 1e-2


def test_c5_fused_cache_write_at_full_size():
    """The decode call that stores the new tokens' rows itself (2048 CTAs store a row and then
    copy the page that holds it, with the memory system saturated) must give, bit for bit, the
    result of a separate cache write followed by the plain call."""
    import lazy_attention_b200 as la
    case = synth.config_c5(device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    bt, seq = case["block_table"].cpu(), case["seq_lens"].cpu()
    slots = torch.tensor([int(bt[b, (int(seq[b]) - 1) // 16]) * 16 + (int(seq[b]) - 1) % 16 for b in range(len(seq))],
                         dtype=torch.int64).cuda()

    def run(slot_mapping, key, value):
        out = util.new_out(case)
        la.chunked_prefill_paged_decode(
            case["q"], key, value, out, case["kv_cache_dtype"], case["k_cache"], case["v_cache"], case["block_table"],
            case["query_start_loc"], case["seq_lens"], case["max_seq_len"], 1, case["k_scale"], case["v_scale"],
            sm_scale=case["sm_scale"], cos_sin_cache=case["cos_sin_cache"], is_lazy=case["is_lazy"],
            q_offset=case["q_offset"], q_mask=case["q_mask"], packed_block_table=case["packed_block_table"],
            kernel="tensor", slot_mapping=slot_mapping)
        torch.cuda.synchronize()
        assert la.device_status() == 0
        return out

    before = run(None, case["k"], case["v"])
    for rep in range(3):
        g = torch.Generator(device="cuda").manual_seed(rep)
        key = (torch.randn(case["k"].shape, generator=g, device="cuda") * 1.2).to(case["k"].dtype)
        value = (torch.randn(case["v"].shape, generator=g, device="cuda") * 1.2).to(case["v"].dtype)
        fused = run(slots, key, value)          # the caches are several GB: written in place, no copies
        la.write_to_paged_cache(key, value, case["k_cache"], case["v_cache"], slots, case["kv_cache_dtype"],
                                case["k_scale"], case["v_scale"])
        separate = run(None, key, value)
        assert torch.equal(fused, separate), f"repetition {rep}: the call did not attend to the rows it stored"
        assert not torch.equal(fused, before)
        before = separate
