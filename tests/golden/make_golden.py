"""Regenerate tests/golden/*.npz from the reference implementation.

Run where a checkout of the reference is available and name it in
``REFERENCE_ROOT``::

    REFERENCE_ROOT=<path to the reference checkout> python tests/golden/make_golden.py

Floating-point fixtures: the reference's own Triton kernels are executed on CPU
tensors through Triton's interpreter (``TRITON_INTERPRET=1``; float32, the only
dtype family the interpreter evaluates faithfully) on small seeded inputs; the
inputs and the kernels' outputs are stored.  Integer fixtures: the reference's
scheduler function is executed from its source text (its module cannot be
imported against the vLLM version installed here) and the reference's
``max_rotation_offset`` is imported directly.

``python tests/golden/make_golden.py int cos_sin backend`` regenerates only the named
groups (the float group runs the Triton interpreter for minutes).

The stored files are what the CPU tests pin the oracle with and what the GPU
tests compare the CUDA kernels against; nothing at test time reads the
reference checkout.
"""
from __future__ import annotations

import ast
import os
import sys
import types
from pathlib import Path
from types import SimpleNamespace

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
sys.dont_write_bytecode = True

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
if "REFERENCE_ROOT" not in os.environ:
    raise SystemExit("set REFERENCE_ROOT to the reference checkout")
REF = Path(os.environ["REFERENCE_ROOT"])
sys.path.insert(0, str(REF / "lazy_attn"))

from lazy_attention_b200 import synth  # noqa: E402

# The dispatch wrappers import a ROCm predicate whose module initialises CUDA;
# give them a stand-in so they import on a GPU-less box.
_stub = types.ModuleType("vllm.platforms.rocm")
_stub.use_rocm_custom_paged_attention = lambda *a, **k: False
sys.modules["vllm.platforms.rocm"] = _stub

from lazy.attention.ops.prefix_prefill import context_attention_fwd as ref_lazy_prefill  # noqa: E402
from lazy.attention.ops.chunked_prefill_paged_decode import chunked_prefill_paged_decode as ref_lazy_op  # noqa: E402
from lazy.attention.old_ops.prefix_prefill import context_attention_fwd as ref_mepic_prefill  # noqa: E402
from lazy.attention.old_ops.chunked_prefill_paged_decode import chunked_prefill_paged_decode as ref_mepic_op  # noqa: E402
from lazy.utils.rotation import MAX_PACKED_Q_OFFSET, max_rotation_offset as ref_max_rot  # noqa: E402

SMALL = synth.Geometry(4, 2, 32, 16, 500000.0)
POOL = [20, 16, 9, 33, 48]


def _np(t):
    if t.dtype == torch.bool:
        return t.numpy().astype(np.uint8)
    return t.numpy()


def _save(name, case, out, extra=None):
    keys = ["q", "k", "v", "k_cache", "v_cache", "block_table", "q_offset", "q_mask", "is_lazy",
            "query_start_loc", "seq_lens", "k_scale", "v_scale", "cos_sin_cache"]
    data = {k: _np(case[k]) for k in keys}
    if "packed_block_table" in case:
        data["packed_block_table"] = _np(case["packed_block_table"])
    data["out"] = out.numpy()
    data["meta"] = np.array([case["geom"].num_q_heads, case["geom"].num_kv_heads,
                             case["geom"].head_dim, case["geom"].block_size,
                             case["max_seq_len"], case["max_query_len"], case["num_tokens"]],
                            dtype=np.int64)
    data["sm_scale"] = np.float32(case["sm_scale"])
    if extra:
        data.update(extra)
    np.savez_compressed(HERE / f"{name}.npz", **data)
    print(f"wrote {name}.npz  out|max|={out.abs().max():.4f}")


def _packed(case):
    bt = case["block_table"].to(torch.int64)
    return (bt << 32) | (case["q_offset"].to(torch.int64) << 16) | case["q_mask"].to(torch.int64)


def _run_lazy_prefill(case, skip_decode=False, sliding_window=None):
    T = case["num_tokens"]
    out = torch.zeros(T, case["geom"].num_q_heads, case["geom"].head_dim, dtype=case["q"].dtype)
    ref_lazy_prefill(case["q"], case["k"], case["v"], out, case["kv_cache_dtype"],
                     case["k_cache"], case["v_cache"], case["block_table"],
                     case["query_start_loc"], case["seq_lens"], case["max_seq_len"],
                     case["max_query_len"], case["k_scale"][0], case["v_scale"][0],
                     sliding_window=sliding_window, sm_scale=case["sm_scale"],
                     skip_decode=skip_decode, cos_sin_cache=case["cos_sin_cache"],
                     rotary_dim=case["geom"].head_dim, is_lazy=case["is_lazy"],
                     q_offset=case["q_offset"], q_mask=case["q_mask"])
    return out


def _run_lazy_op(case, sliding_window=None, alibi=None):
    T = case["num_tokens"]
    out = torch.zeros(T, case["geom"].num_q_heads, case["geom"].head_dim, dtype=case["q"].dtype)
    case["packed_block_table"] = _packed(case)
    ref_lazy_op(query=case["q"], key=case["k"], value=case["v"], output=out,
                kv_cache_dtype=case["kv_cache_dtype"], key_cache=case["k_cache"],
                value_cache=case["v_cache"], block_table=case["block_table"],
                query_start_loc=case["query_start_loc"], seq_lens=case["seq_lens"],
                max_seq_len=case["max_seq_len"], max_query_len=case["max_query_len"],
                k_scale=case["k_scale"][0], v_scale=case["v_scale"][0], alibi_slopes=alibi,
                sliding_window=sliding_window, sm_scale=case["sm_scale"],
                rotary_dim=case["geom"].head_dim, cos_sin_cache=case["cos_sin_cache"],
                is_lazy=case["is_lazy"], lazy_variant=None, q_offset=case["q_offset"],
                q_mask=case["q_mask"], packed_block_table=case["packed_block_table"])
    return out


def _run_mepic_op(case, is_mepic=True):
    T = case["num_tokens"]
    out = torch.zeros(T, case["geom"].num_q_heads, case["geom"].head_dim, dtype=case["q"].dtype)
    ref_mepic_op(query=case["q"], key=case["k"], value=case["v"], output=out,
                 kv_cache_dtype=case["kv_cache_dtype"], key_cache=case["k_cache"],
                 value_cache=case["v_cache"], block_table=case["block_table"],
                 query_start_loc=case["query_start_loc"], seq_lens=case["seq_lens"],
                 max_seq_len=case["max_seq_len"], max_query_len=case["max_query_len"],
                 k_scale=case["k_scale"][0], v_scale=case["v_scale"][0],
                 sm_scale=case["sm_scale"], rotary_dim=case["geom"].head_dim,
                 cos_sin_cache=case["cos_sin_cache"], q_offset=case["q_offset"],
                 q_mask=case["q_mask"], is_mepic=is_mepic)
    return out


MIXED = [dict(docs=[2, 0, 1], qlen=5), dict(docs=[3, 1], qlen=19),
         dict(docs=[0], qlen=7, lazy=False), dict(docs=[1, 2, 4], qlen=1),
         dict(docs=[4, 3], qlen=1), dict(docs=[2], qlen=1, lazy=False)]


def gen_float():
    # 1. lazy prefill kernel alone (decode rows untouched through skip_decode)
    case = synth.build_prefill(SMALL, torch.float32, POOL, MIXED, seed=11)
    _save("lazy_prefill_small", case, _run_lazy_prefill(case, skip_decode=True))
    # 2. lazy dispatch wrapper on a mixed batch: prefill kernel + decode kernel
    case = synth.build_prefill(SMALL, torch.float32, POOL, MIXED, seed=12)
    _save("lazy_mixed_small", case, _run_lazy_op(case))
    # 3. per-token wrapper on a mixed batch
    case = synth.build_prefill(SMALL, torch.float32, POOL, MIXED, seed=13, variant="mepic")
    _save("mepic_mixed_small", case, _run_mepic_op(case, True))
    # 4. per-token wrapper with is_mepic=False (page offset + in-page index)
    case = synth.build_prefill(SMALL, torch.float32, POOL, MIXED, seed=14, variant="lazy")
    _save("mepic_off_mixed_small", case, _run_mepic_op(case, False))
    # 5. fp8 e4m3 cache, float32 activations.  The reference's rotating prefill
    #    branches cannot be compiled with an fp8 cache (they name an undefined
    #    variable on the V dequantisation line, ops/prefix_prefill.py:313), so
    #    the fixtures cover what the reference can run: decode (rotating and
    #    plain sequences) and the plain prefill branch.
    dec8 = [dict(docs=[1, 2, 4], qlen=1), dict(docs=[0, 3], qlen=1), dict(docs=[2], qlen=1, lazy=False)]
    case = synth.build_prefill(SMALL, torch.float32, POOL, dec8, seed=15, kv_dtype="fp8_e4m3",
                               k_scale=0.11, v_scale=0.07)
    _save("lazy_decode_fp8_small", case, _run_lazy_op(case))
    pre8 = [dict(docs=[2, 0, 1], qlen=5, lazy=False), dict(docs=[3], qlen=19, lazy=False)]
    case = synth.build_prefill(SMALL, torch.float32, POOL, pre8, seed=19, kv_dtype="fp8_e4m3",
                               k_scale=0.13, v_scale=0.09)
    _save("plain_prefill_fp8_small", case, _run_lazy_prefill(case))
    # 6. sliding window
    case = synth.build_prefill(SMALL, torch.float32, POOL, MIXED, seed=16)
    _save("lazy_mixed_window_small", case, _run_lazy_op(case, sliding_window=24),
          extra=dict(sliding_window=np.int64(24)))
    # 7. decode only with alibi slopes
    dec = [dict(docs=[1, 2, 4], qlen=1), dict(docs=[0, 3], qlen=1), dict(docs=[2], qlen=1, lazy=False)]
    case = synth.build_prefill(SMALL, torch.float32, POOL, dec, seed=17)
    slopes = torch.tensor([0.5, 0.25, 0.125, 0.0625], dtype=torch.float32)
    _save("lazy_decode_alibi_small", case, _run_lazy_op(case, alibi=slopes),
          extra=dict(alibi_slopes=slopes.numpy()))
    # 8. plain (unscaled) rope table, head_dim 64, page size 8
    g2 = synth.Geometry(6, 2, 64, 8, 10000.0)
    case = synth.build_prefill(g2, torch.float32, [10, 8, 23], [dict(docs=[1, 2, 0], qlen=9),
                                                                dict(docs=[2, 0], qlen=1)],
                               seed=18, llama3=False)
    _save("lazy_mixed_bs8_small", case, _run_lazy_op(case))
    # 9. the first benchmark configuration (1B geometry, fp32, batch 2, 3x128 docs, 32 new)
    for variant in ("lazy", "mepic"):
        case = synth.config_c1(variant=variant)
        if variant == "lazy":
            out = _run_lazy_prefill(case)
        else:
            out = _run_mepic_op(case, True)
        heads = [0, 5, 13, 31]
        data = dict(out_heads=out[:, heads].numpy(), heads=np.array(heads),
                    q_checksum=np.float64(case["q"].double().sum().item()),
                    kc_checksum=np.float64(case["k_cache"].double().sum().item()))
        np.savez_compressed(HERE / f"c1_{variant}.npz", **data)
        print(f"wrote c1_{variant}.npz")


def _load_scheduler_fn(name):
    """Execute one top-level function of the reference scheduler from its source."""
    src = (REF / "lazy_attn/lazy/core/sched/scheduler.py").read_text()
    tree = ast.parse(src)
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"np": np, "Request": object}
            exec(compile(mod, "scheduler.py", "exec"), ns)
            return ns[name]
    raise KeyError(name)


def gen_int():
    fn = _load_scheduler_fn("metadata_for_lazy_attention")
    rng = np.random.default_rng(5)
    cases = [([6, 15, 8, 2], 8), ([6], 16), ([16, 16], 16), ([1, 1, 1, 1, 1], 16),
             ([4096, 17], 16), ([100] * 32, 16), ([1024] * 64, 16), ([1] * 8, 16), ([], 16)]
    for _ in range(24):
        n = int(rng.integers(1, 12))
        cases.append(([int(v) for v in rng.integers(1, 700, size=n)], int(rng.choice([8, 16, 32]))))
    rec = []
    for lens, bs in cases:
        padded = [(v + bs - 1) // bs * bs for v in lens]
        off, msk = fn(SimpleNamespace(document_lens=lens, document_lens_padded=padded), bs)
        rec.append(dict(lens=lens, padded=padded, bs=bs, q_offset=[int(v) for v in off],
                        q_mask=[int(v) for v in msk], max_rot=int(ref_max_rot(lens, padded))))
    import json
    (HERE / "metadata_vectors.json").write_text(json.dumps(
        dict(max_packed_q_offset=int(MAX_PACKED_Q_OFFSET), cases=rec)))
    print("wrote metadata_vectors.json", len(rec))


def gen_cos_sin():
    """Rows of the reference's own llama3 cos/sin mirror (model_executor/rope/cos_sin.py:127-148),
    for the geometries of the benchmark configurations."""
    from lazy.model_executor.rope.cos_sin import llama3_cos_sin_torch
    positions = [0, 1, 2, 17, 511, 4097, 65024, 65535, 131071]
    data = {"positions": np.array(positions, dtype=np.int64),
            "params": np.array([500000.0, 8.0, 1.0, 4.0, 8192.0], dtype=np.float64)}
    for head in (64, 128):
        cos, sin = zip(*[llama3_cos_sin_torch(pos, head, 500000.0, 8.0, 1.0, 4.0, 8192, "cpu") for pos in positions])
        data[f"cos_{head}"] = torch.stack(cos).numpy()
        data[f"sin_{head}"] = torch.stack(sin).numpy()
    np.savez_compressed(HERE / "cos_sin_llama3.npz", **data)
    print("wrote cos_sin_llama3.npz")


def gen_backend_keywords():
    """What the reference's attention backend imports and which keyword arguments it passes to
    the two operators (backends/triton_attn.py), read from its source text: the patch-in test
    binds the replacement operators against exactly these sets."""
    import json
    src = (REF / "lazy_attn/lazy/attention/backends/triton_attn.py").read_text()
    tree = ast.parse(src)
    imports = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom) and node.module and "chunked_prefill_paged_decode" in node.module:
            for alias in node.names:
                imports[alias.asname or alias.name] = "." * node.level + node.module
    common, updates = [], []
    for node in ast.walk(tree):
        if isinstance(node, ast.Assign) and isinstance(node.value, ast.Call) and \
                getattr(node.value.func, "id", "") == "dict" and \
                any(getattr(t, "id", "") == "kernel_kwargs" for t in node.targets):
            common = [k.arg for k in node.value.keywords]
    for node in ast.walk(tree):
        if isinstance(node, ast.If):
            for branch in (node.body, node.orelse):
                upd, callee = None, None
                for stmt in branch:
                    call = stmt.value if isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Call) else None
                    if call is None:
                        continue
                    f = call.func
                    if isinstance(f, ast.Attribute) and f.attr == "update" and getattr(f.value, "id", "") == "kernel_kwargs":
                        upd = [k.arg for k in call.keywords]
                    elif isinstance(f, ast.Name) and f.id.startswith("chunked_prefill_paged_decode"):
                        callee = f.id
                if upd is not None and callee is not None:
                    updates.append((callee, upd))
    rec = dict(imports=imports, common=common, extra={c: u for c, u in updates})
    assert set(rec["extra"]) == {"chunked_prefill_paged_decode", "chunked_prefill_paged_decode_old"}, rec
    (HERE / "backend_keywords.json").write_text(json.dumps(rec, indent=1))
    print("wrote backend_keywords.json", {k: len(v) for k, v in rec["extra"].items()}, len(common))


if __name__ == "__main__":
    only = sys.argv[1:]
    if not only or "int" in only:
        gen_int()
    if not only or "cos_sin" in only:
        gen_cos_sin()
    if not only or "backend" in only:
        gen_backend_keywords()
    if not only or "float" in only:
        gen_float()
