"""Edge cases of sizes and table fields, tensor-core / split-KV kernels and the general kernel
against the oracle: a decode batch behind ~61k cached tokens (rotation offsets far above 32767),
pages that are padding from the first slot on, sequences without any cached context, and
one-token requests through the prefill operator."""
import pytest
import torch

import util
from lazy_attention_b200 import synth

pytestmark = pytest.mark.gpu

HALF = dict(atol=2e-2, rtol=1e-2)
FP8 = dict(atol=5e-2, rtol=1e-2)
POOL = [100, 64, 33, 250, 16, 129]


@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
@pytest.mark.parametrize("variant,op", [("lazy", "lazy_op"), ("mepic", "mepic_op")])
def test_decode_behind_sixty_thousand_tokens(kv, variant, op):
    docs = [[512] * 120, [512] * 70 + [100, 37], [300] * 3]
    scales = dict(k_scale=0.12, v_scale=0.08) if "fp8" in kv else {}
    case = synth.build_decode(synth.GEOM_8B, torch.bfloat16, docs, seed=41, device="cuda", kv_dtype=kv,
                              variant=variant, **scales)
    if variant == "lazy":
        assert int(case["q_offset"].max()) > 40000
    case["packed_block_table"] = util.pack_host(case).cuda()
    want = util.run_oracle(case, op)
    for kernel in ("tensor", "general"):
        got = util.run_cuda(case, op, kernel=kernel)
        util.assert_close(got, want, what=f"long decode {kv} {variant} {kernel}", **(FP8 if "fp8" in kv else HALF))


@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
def test_pages_that_are_all_padding(kv):
    """q_mask = 16 on some pages (every slot is padding), next to partly padded ones."""
    reqs = [dict(docs=[2, 0, 1], qlen=130), dict(docs=[3, 1, 4], qlen=1), dict(docs=[5, 4], qlen=40)]
    ks, vs = (0.11, 0.07) if "fp8" in kv else (1.0, 1.0)
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, POOL, reqs, seed=19, variant="lazy", device="cuda",
                               kv_dtype=kv, k_scale=ks, v_scale=vs)
    ctx_pages = ((case["seq_lens"] - (case["query_start_loc"][1:] - case["query_start_loc"][:-1])) // 16).cpu()
    for b in range(len(reqs)):
        n = int(ctx_pages[b])
        case["q_mask"][b, 1] = 16
        case["q_mask"][b, n // 2] = 16
        case["q_mask"][b, n - 1] = 16   # the last whole page of the context
    # a whole 128-key tile of padding at the start of a request (its running maximum starts at
    # -inf) and in the middle of a decode row (whole tiles of the split-KV kernel)
    case["q_mask"][0, 0:8] = 16
    case["q_mask"][1, 8:16] = 16
    case["packed_block_table"] = util.pack_host(case).cuda()
    want = util.run_oracle(case, "lazy_op")
    for kernel in ("tensor", "general"):
        got = util.run_cuda(case, "lazy_op", kernel=kernel)
        util.assert_close(got, want, what=f"all-padding pages {kv} {kernel}", **(FP8 if "fp8" in kv else HALF))


@pytest.mark.parametrize("variant,op", [("lazy", "lazy_op"), ("mepic", "mepic_op")])
def test_sequences_without_cached_context(variant, op):
    """Decode rows and prefill requests whose only keys are their own new tokens."""
    reqs = [dict(docs=[], qlen=1), dict(docs=[], qlen=300), dict(docs=[2], qlen=1), dict(docs=[], qlen=17)]
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, POOL, reqs, seed=23, variant=variant, device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    want = util.run_oracle(case, op)
    for kernel in ("tensor", "general"):
        got = util.run_cuda(case, op, kernel=kernel)
        util.assert_close(got, want, what=f"no context {variant} {kernel}", **HALF)


def test_one_token_requests_through_the_prefill_operator():
    """context_attention_fwd with skip_decode off computes one-token requests itself."""
    reqs = [dict(docs=[2, 0], qlen=1), dict(docs=[3, 1, 5], qlen=260), dict(docs=[4], qlen=1)]
    case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, POOL, reqs, seed=29, variant="lazy", device="cuda")
    case["packed_block_table"] = util.pack_host(case).cuda()
    want = util.run_oracle(case, "lazy_prefill")
    for kernel in ("tensor", "general"):
        got = util.run_cuda(case, "lazy_prefill", kernel=kernel)
        util.assert_close(got, want, what=f"one-token requests {kernel}", **HALF)


def test_calls_on_two_streams_keep_their_partial_results_apart(monkeypatch):
    """Two split-KV calls in flight on two streams: each stream has its own scratch, so the
    results equal those of the calls run one after the other."""
    monkeypatch.setenv("LAZY_ATTN_B200_PREFILL_SPLITS", "4")
    cases = []
    for seed in (51, 52):
        reqs = [dict(docs=[2, 0, 1, 3, 5], qlen=300), dict(docs=[3, 1, 5, 0], qlen=260)]
        case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, [700, 640, 333, 900, 160, 1290], reqs, seed=seed,
                                   variant="lazy", device="cuda")
        case["packed_block_table"] = util.pack_host(case).cuda()
        cases.append(case)
    alone = [util.run_cuda(c, "lazy_prefill", kernel="tensor") for c in cases]
    import lazy_attention_b200 as la
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [util.new_out(c) for c in cases]
    torch.cuda.synchronize()
    for _ in range(20):
        for c, o, s in zip(cases, outs, streams):
            with torch.cuda.stream(s):
                la.context_attention_fwd(c["q"], c["k"], c["v"], o, c["kv_cache_dtype"], c["k_cache"], c["v_cache"],
                                         c["block_table"], c["query_start_loc"], c["seq_lens"], c["max_seq_len"],
                                         c["max_query_len"], c["k_scale"], c["v_scale"], sm_scale=c["sm_scale"],
                                         cos_sin_cache=c["cos_sin_cache"], is_lazy=c["is_lazy"], q_offset=c["q_offset"],
                                         q_mask=c["q_mask"], kernel="tensor")
    torch.cuda.synchronize()
    assert la.device_status() == 0
    for o, a in zip(outs, alone):
        assert torch.equal(o.float().cpu(), a), "a call's result changed when another stream's call ran beside it"


def test_per_token_operator_with_absolute_rotation_off_at_large_offsets():
    """``is_mepic=False`` rotates a page's tokens at ``q_offset - 1 + slot``: offsets far above
    32767, D = 128 and 64, through the prefill operator and the dispatch operator."""
    for geom in (synth.GEOM_8B, synth.GEOM_1B):
        reqs = [dict(docs=[2, 0, 1], qlen=130), dict(docs=[5, 4], qlen=40)]
        case = synth.build_prefill(geom, torch.bfloat16, POOL, reqs, seed=31, variant="mepic", device="cuda",
                                   max_position=65536)
        off = case["q_offset"]
        for b in range(off.shape[0]):
            pages = int((case["seq_lens"][b] - (case["query_start_loc"][b + 1] - case["query_start_loc"][b])) // 16)
            off[b, :pages] = torch.randint(30000, 65000, (pages,), generator=torch.Generator().manual_seed(b)).to(off)
        want = util.run_oracle(case, "mepic_prefill", is_mepic=False)
        for kernel in ("tensor", "general"):
            got = util.run_cuda(case, "mepic_prefill", kernel=kernel, is_mepic=False)
            util.assert_close(got, want, what=f"absolute rotation off, d{geom.head_dim}, {kernel}", **HALF)


@pytest.mark.parametrize("dtype,kv", [(torch.float16, "auto"), (torch.float16, "fp8_e5m2"), (torch.bfloat16, "fp8_e5m2")])
def test_long_decode_at_head_dim_64(dtype, kv):
    """1B geometry (1 KB fp8 pages: four pages per tile), contexts up to ~40k tokens."""
    docs = [[512] * 80, [700] * 9 + [33], [16] * 5, [2048] * 12]
    scales = dict(k_scale=0.12, v_scale=0.08) if "fp8" in kv else {}
    case = synth.build_decode(synth.GEOM_1B, dtype, docs, seed=43, device="cuda", kv_dtype=kv, **scales)
    case["packed_block_table"] = util.pack_host(case).cuda()
    want = util.run_oracle(case, "lazy_op")
    for kernel in ("tensor", "general"):
        got = util.run_cuda(case, "lazy_op", kernel=kernel)
        util.assert_close(got, want, what=f"long decode d64 {dtype} {kv} {kernel}", **(FP8 if "fp8" in kv else HALF))
