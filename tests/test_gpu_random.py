"""Seeded random batches through the tensor-core / split-KV kernels against the oracle.

Each case draws a geometry, a document pool, and a mixed batch (prefill requests of ragged
lengths, decode rows, requests without context, plain and rotating requests, documents whose
last page is partly padding) and runs it with the planner's own split count and with a pinned one, so that the CTA
pairs, the single-CTA kernel, the merge kernel and the masks of ragged tiles all meet
shapes nobody wrote down by hand.  Tolerance: bf16 / fp16 2e-2 absolute, 1e-2 relative.
"""
import numpy as np
import pytest
import torch

import util
from lazy_attention_b200 import synth

pytestmark = pytest.mark.gpu

HALF = dict(atol=2e-2, rtol=1e-2)
FP8 = dict(atol=5e-2, rtol=1e-2)


def _draw(seed):
    rng = np.random.default_rng(seed)
    hkv = int(rng.choice([1, 2, 4, 8]))
    group = int(rng.choice([1, 2, 4, 8]))
    geom = synth.Geometry(hkv * group, hkv, int(rng.choice([64, 128])))
    pool = [int(n) for n in rng.integers(1, 400, size=int(rng.integers(2, 7)))]
    reqs = []
    for _ in range(int(rng.integers(1, 6))):
        kind = rng.random()
        ndocs = int(rng.integers(0, min(4, len(pool)) + 1))
        docs = [int(d) for d in rng.choice(len(pool), size=ndocs, replace=False)]
        if kind < 0.2:
            qlen = 1
        elif kind < 0.6:
            qlen = int(rng.integers(2, 140))
        else:
            qlen = int(rng.integers(140, 700))
        reqs.append(dict(docs=docs, qlen=qlen, lazy=bool(rng.random() < 0.75)))
    dtype = torch.bfloat16 if rng.random() < 0.7 else torch.float16
    kv = "auto" if rng.random() < 0.7 else "fp8_e4m3"
    variant = "lazy" if rng.random() < 0.6 else "mepic"
    return geom, pool, reqs, dtype, kv, variant


@pytest.mark.parametrize("seed", list(range(24)))
@pytest.mark.parametrize("splits", [None, 3])
def test_random_mixed_batches(seed, splits, monkeypatch):
    geom, pool, reqs, dtype, kv, variant = _draw(seed)
    if splits is not None:
        monkeypatch.setenv("LAZY_ATTN_B200_PREFILL_SPLITS", str(splits))
    ks, vs = (0.11, 0.07) if "fp8" in kv else (1.0, 1.0)
    case = synth.build_prefill(geom, dtype, pool, reqs, seed=100 + seed, variant=variant, device="cuda",
                               kv_dtype=kv, k_scale=ks, v_scale=vs)
    case["packed_block_table"] = util.pack_host(case).cuda()
    op = "lazy_op" if variant == "lazy" else "mepic_op"
    got = util.run_cuda(case, op, kernel="tensor")
    want = util.run_oracle(case, op)
    what = f"seed {seed}: heads {geom.num_q_heads}/{geom.num_kv_heads} d{geom.head_dim} {dtype} {kv} {variant} " \
           f"qlens {[r['qlen'] for r in reqs]} splits {splits}"
    util.assert_close(got, want, what=what, **(FP8 if "fp8" in kv else HALF))


def _draw_decode(seed):
    rng = np.random.default_rng(1000 + seed)
    hkv = int(rng.choice([1, 2, 4, 8]))
    group = int(rng.choice([1, 2, 4, 8]))
    geom = synth.Geometry(hkv * group, hkv, int(rng.choice([64, 128])))
    docs = []
    for _ in range(int(rng.integers(1, 9))):
        n = int(rng.integers(1, 7))
        # short, ragged and a few long documents: contexts from a handful of tokens to ~12k
        docs.append([int(x) for x in np.where(rng.random(n) < 0.2, rng.integers(1500, 3000, n), rng.integers(1, 400, n))])
    dtype = torch.bfloat16 if rng.random() < 0.7 else torch.float16
    kv = "auto" if rng.random() < 0.5 else "fp8_e4m3"
    variant = "lazy" if rng.random() < 0.6 else "mepic"
    flags = [bool(rng.random() < 0.8) for _ in docs]
    return geom, docs, dtype, kv, variant, flags


@pytest.mark.parametrize("seed", list(range(24)))
@pytest.mark.parametrize("chunk", [None, 16])
def test_random_decode_batches(seed, chunk, monkeypatch):
    """Decode-only batches through the split-KV kernel, with the planner's run length and with the
    shortest one (many splits per sequence, the last split walking on to the real last page)."""
    geom, docs, dtype, kv, variant, flags = _draw_decode(seed)
    if chunk is not None:
        monkeypatch.setenv("LAZY_ATTN_B200_DECODE_CHUNK", str(chunk))
    ks, vs = (0.13, 0.09) if "fp8" in kv else (1.0, 1.0)
    case = synth.build_decode(geom, dtype, docs, seed=200 + seed, device="cuda", kv_dtype=kv, variant=variant,
                              k_scale=ks, v_scale=vs, lazy_flags=flags)
    case["packed_block_table"] = util.pack_host(case).cuda()
    op = "lazy_op" if variant == "lazy" else "mepic_op"
    got = util.run_cuda(case, op, kernel="tensor")
    want = util.run_oracle(case, op)
    what = f"decode seed {seed}: heads {geom.num_q_heads}/{geom.num_kv_heads} d{geom.head_dim} {dtype} {kv} " \
           f"{variant} contexts {[sum(d) for d in docs]} chunk {chunk}"
    util.assert_close(got, want, what=what, **(FP8 if "fp8" in kv else HALF))
