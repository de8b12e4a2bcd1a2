#!/usr/bin/env python
"""Benchmark of the deferred-RoPE attention path on synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c5|c3|c2]
                    [--impl ours|reference] [--kernel auto|general|tensor]

A step is one attention-layer call over one batch.  Workloads are the
BASELINE configurations (seeded synthetic inputs of their shapes):

  c4 (default)  prefix-prefill, 8B geometry, bf16, 8 requests x 65536 cached
                tokens (128 documents x 512 at random slots) + 512 new tokens;
                N > 1 shards by KV-head group and gathers the outputs.
  c5            decode, 8B geometry, 256 sequences x 4k..16k cached tokens,
                e4m3 KV, bf16 query; N > 1 shards by request.
  c3, c2        the smaller prefill configurations (1 GPU).

One JSON line is printed by rank 0: the headline workload (c4 unless
``--workload`` says otherwise) with, under ``also``, the decode workload c5 at
the same N (sharded by request) and, at N = 1, the ragged prefill workload c3 and
the small one c2 (the prefill shape the reference's Triton kernel compiles for on
this GPU), each with its own value, roofline and end-to-end figure.  At N = 1 the line
also carries ``triton_baseline``: the reference's own Triton kernels compiled
for this GPU and timed on the same inputs (outside every timed region of this
library).  At N > 1 one step of the output gather fused into the kernels is
compared bit for bit with the same kernels followed by an NCCL all-gather
before anything is timed (``gather_check``; a mismatch ends the run non-zero).

``value`` is query tokens per second of the whole job with all inputs resident
in HBM (the call's launches replayed from a CUDA graph unless ``--cuda-graph
off``; the eager cost of the same call through the Python wrapper is reported
beside it as ``execution.eager_ms_per_step``).  A call sharded by KV-head group
processes every token on every rank, so its tokens are counted once, not once
per rank.  ``e2e`` is the same call through the public API with the step's
activations and metadata copied from pinned host memory and the result copied
back, every step - measured in sequence on one stream and as a three-stream
pipeline over two buffer sets, the better of the two reported; at N > 1 every
rank uploads its own shard and reads back its 1/N slice of the gathered rows,
so the job reads the result back once.  Timing is CUDA events on the launching
stream, max over ranks.  ``speedup_vs_ideal`` is the time the whole job's
algorithmic work, spread evenly over the N ranks, would take at the measured peak,
divided by rank 0's kernel time (at N = 1 it equals ``roofline.frac``).

``--impl reference`` times the CPU oracle (a float32 torch restatement of the
reference kernels) with all host threads; each step is one call over a bounded
sample of the workload made of whole requests / sequences with their full
context, so its tokens per second need no extrapolation.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "deferred-RoPE attention throughput (query tokens/s per attention-layer call)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c4", choices=["c2", "c3", "c4", "c5"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel", default="auto", choices=["auto", "general", "tensor"])
    ap.add_argument("--variant", default="lazy", choices=["lazy", "mepic"])
    ap.add_argument("--kv-dtype", default="auto", choices=["auto", "bf16", "fp8_e4m3", "fp8_e5m2"],
                    help="cache dtype of the c4 / c5 workload ('auto' = the quoted configuration: bf16 for c4, "
                         "e4m3 for c5)")
    ap.add_argument("--scale", type=float, default=1.0,
                    help="shrink the workload (profiling captures only; not a bench value)")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="on ONE GPU, run the shard a rank of an N-GPU job would get (tuning aid for the "
                         "per-rank kernel; not a bench value)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="only the headline workload")
    ap.add_argument("--no-triton", action="store_true", help="skip the Triton reference leg")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: 'fused' = the kernels store their result rows into every rank's output "
                         "buffer (peer-mapped memory) and the step ends with a barrier; 'nccl' = all-gather")
    ap.add_argument("--barrier", default="signal", choices=["signal", "nccl"],
                    help="how a step of the fused gather ends: 'signal' = the library's own kernel (every rank "
                         "announces itself in its peers' signal buffers and waits for theirs), 'nccl' = a "
                         "one-element all-reduce")
    ap.add_argument("--cuda-graph", default="on", choices=["on", "off"],
                    help="replay the library's launches of one call from a CUDA graph in the device-resident "
                         "timing (the end-to-end leg always launches eagerly)")
    return ap.parse_args()


# --------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------
def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), tf_burst=float(d["bf16_tflops"]),
                    tf_sust=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sust=1400.0, src="fallback")


def recorded_traffic(name):
    """DRAM bytes per launch of the workload's dominant kernel as recorded in the ncu summary
    under profiles/ (a line ``dram_traffic_bytes_per_launch[<workload>]: <number>``), or None."""
    pat = re.compile(r"dram_traffic_bytes_per_launch\[" + re.escape(name) + r"\]\s*:\s*([0-9.eE+]+)")
    for f in sorted((ROOT / "profiles").glob("*.md")):
        m = pat.search(f.read_text())
        if m:
            return float(m.group(1))
    return None


L2_LARGE = "inputs larger than L2 (no flush)"
L2_SMALL = "inputs smaller than L2: flushed by a 256 MB write between steps"


def workload_info(name, world=1, scale=1.0, kv_dtype="auto"):
    """Description of a workload (no tensors): the `config.workload` text and how it shards."""
    if name == "c4":
        ndocs = max(1, int(round(128 * scale)))
        return dict(kind="prefill", workload=f"c4: 8B geometry bf16, 8 requests x {ndocs}x512 cached "
                    f"tokens + 512 new, block 16" + ("" if kv_dtype == "auto" else f", {kv_dtype} cache")
                    + ("" if scale == 1.0 else f" (scaled {scale})"),
                    partition="kv_head_group" if world > 1 else "none", scaling="strong", full_heads=(32, 8),
                    l2=L2_LARGE)
    if name == "c3":
        return dict(kind="prefill", workload="c3: 8B geometry bf16, 32 requests x 20 docs U{256..1024} "
                    "Zipf(1.1) from a 200-doc pool, 64..256 new tokens", partition="none",
                    scaling="strong", full_heads=(32, 8), l2=L2_LARGE)
    if name == "c2":
        return dict(kind="prefill", workload="c2: 1B geometry bf16, 1 request x 10x512 cached tokens + 128 new",
                    partition="none", scaling="strong", full_heads=(32, 8), l2=L2_SMALL)
    if name == "c5":
        nseq = max(world, int(round(256 * scale)))
        return dict(kind="decode", workload=f"c5: 8B geometry decode, {nseq} sequences x 4k..16k cached tokens, "
                    f"{'e4m3' if kv_dtype == 'auto' else kv_dtype} KV, bf16 query, block 16",
                    partition="request" if world > 1 else "none", scaling="strong", full_heads=(32, 8),
                    total_seqs=nseq, l2=L2_LARGE)
    raise KeyError(name)


def c5_documents(nseq):
    """Document lists and cache scales of the decode workload (seeded)."""
    import numpy as np
    rng = np.random.default_rng(0)
    docs = [[512] * int(rng.integers(8, 33)) for _ in range(nseq)]
    ks, vs = float(rng.uniform(0.05, 0.2)), float(rng.uniform(0.05, 0.2))
    return docs, ks, vs


def build_workload(name, device, variant, rank=0, world=1, scale=1.0, kv_dtype="auto"):
    """Returns (case, info).  For world > 1 the returned case is this rank's shard."""
    from lazy_attention_b200 import synth
    if name == "c4":
        batch = 8
        ndocs = max(1, int(round(128 * scale)))
        geom = synth.GEOM_8B
        if world > 1:
            geom = synth.Geometry(geom.num_q_heads // world, geom.num_kv_heads // world,
                                  geom.head_dim, geom.block_size, geom.rope_theta)
        case = synth.config_c4(device=device, variant=variant, batch=batch, num_docs=ndocs, geom=geom,
                               kv_dtype="auto" if kv_dtype == "bf16" else kv_dtype)
    elif name == "c3":
        case = synth.config_c3(device=device, variant=variant)
    elif name == "c2":
        case = synth.config_c2(device=device, variant=variant)
    elif name == "c5":
        nseq = max(world, int(round(256 * scale)))
        docs, ks, vs = c5_documents(nseq)
        mine = list(range(nseq))
        if world > 1:
            from lazy_attention_b200.sharding import lpt_assign
            mine = lpt_assign([sum(d) + 1 for d in docs], world)[rank]
            docs = [docs[i] for i in mine]
        kvd = "fp8_e4m3" if kv_dtype == "auto" else ("auto" if kv_dtype == "bf16" else kv_dtype)
        case = synth.build_decode(synth.GEOM_8B, torch.bfloat16, docs, seed=rank, device=device,
                                  kv_dtype=kvd, variant=variant, k_scale=ks, v_scale=vs)
        case["global_rows"] = mine
    else:
        raise KeyError(name)
    return case, workload_info(name, world, scale, kv_dtype)


def algorithmic_work(case, info):
    """FLOPs and bytes one call must do/move, and the query tokens it serves (this rank's shard)."""
    g = case["geom"]
    Hq, Hkv, D, BS = g.num_q_heads, g.num_kv_heads, g.head_dim, g.block_size
    e_q = case["q"].element_size()
    e_kv = case["k_cache"].element_size()
    flops = 0.0
    byts = 0.0
    if info["kind"] == "prefill":
        for C, Cv, Q in zip(case["ctx_lens"], case["true_ctx"], case["q_lens"]):
            flops += 4.0 * Hq * D * (Q * Cv + Q * (Q + 1) / 2)
            byts += 2.0 * C * Hkv * D * e_kv + 2.0 * Q * Hkv * D * e_q + 2.0 * Q * Hq * D * e_q
            byts += 12.0 * (C / BS + 1)
        units = sum(case["q_lens"])
    else:
        for L in case["seq_lens"].cpu().tolist():
            flops += 4.0 * Hq * D * L
            byts += 2.0 * L * Hkv * D * e_kv + 2.0 * Hq * D * e_q + 8.0 * ((L + BS) // BS)
        units = len(case["seq_lens"])
    return flops, byts, units


# --------------------------------------------------------------------------------------
# one step
# --------------------------------------------------------------------------------------
def make_step(case, info, kernel):
    import lazy_attention_b200 as la
    g = case["geom"]
    out = torch.empty(case["num_tokens"], g.num_q_heads, g.head_dim, dtype=case["q"].dtype,
                      device=case["q"].device)
    common = dict(kv_cache_dtype=case["kv_cache_dtype"], max_seq_len=case["max_seq_len"],
                  k_scale=case["k_scale"], v_scale=case["v_scale"], sm_scale=case["sm_scale"],
                  cos_sin_cache=case["cos_sin_cache"], rotary_dim=g.head_dim, kernel=kernel)
    lazy = case["variant"] == "lazy"

    def step(q=None, k=None, v=None, tables=None, out_=None, peer_out=None):
        o = out if out_ is None else out_
        q_ = case["q"] if q is None else q
        k_ = case["k"] if k is None else k
        v_ = case["v"] if v is None else v
        t = tables or case
        if info["kind"] == "prefill":
            if lazy:
                la.context_attention_fwd(q_, k_, v_, o, k_cache=case["k_cache"], v_cache=case["v_cache"],
                                         b_loc=t["block_table"], b_start_loc=t["query_start_loc"],
                                         b_seq_len=t["seq_lens"], max_input_len=case["max_query_len"],
                                         is_lazy=t["is_lazy"], q_offset=t["q_offset"], q_mask=t["q_mask"],
                                         peer_out=peer_out, **common)
            else:
                la.context_attention_fwd_mepic(q_, k_, v_, o, k_cache=case["k_cache"],
                                               v_cache=case["v_cache"], b_loc=t["block_table"],
                                               b_start_loc=t["query_start_loc"], b_seq_len=t["seq_lens"],
                                               max_input_len=case["max_query_len"], q_offset=t["q_offset"],
                                               q_mask=t["q_mask"], peer_out=peer_out, **common)
        else:
            if lazy:
                la.chunked_prefill_paged_decode(q_, k_, v_, o, key_cache=case["k_cache"],
                                                value_cache=case["v_cache"], block_table=t["block_table"],
                                                query_start_loc=t["query_start_loc"], seq_lens=t["seq_lens"],
                                                max_query_len=1, is_lazy=t["is_lazy"], q_offset=t["q_offset"],
                                                q_mask=t["q_mask"], packed_block_table=t["packed_block_table"],
                                                peer_out=peer_out, **common)
            else:
                la.chunked_prefill_paged_decode_mepic(q_, k_, v_, o, key_cache=case["k_cache"],
                                                      value_cache=case["v_cache"], block_table=t["block_table"],
                                                      query_start_loc=t["query_start_loc"],
                                                      seq_lens=t["seq_lens"], max_query_len=1,
                                                      q_offset=t["q_offset"], q_mask=t["q_mask"],
                                                      peer_out=peer_out, **common)
        return o

    return step, out


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region (queries only)."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(int(float(r[0])))
                mx = max(mx, int(float(r[1])))
                for n, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=mx or None, reasons=sorted(reasons),
                    samples=len(sm))


_flush_buf = None


def flush_l2(device):
    """Evict L2 by writing a buffer twice its size."""
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    _flush_buf.fill_(1)


def time_steps(fn, steps, warmup, device, world, flush=False):
    """CUDA-event time of `steps` calls after `warmup` (events bracket each call, so an
    optional L2 flush between calls is not counted); returns total ms (max over ranks)
    and the per-call ms of this rank."""
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(device)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        if flush:
            flush_l2(device)
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(device)
    per = [starts[i].elapsed_time(ends[i]) for i in range(steps)]
    total = sum(per) if flush else starts[0].elapsed_time(ends[-1])
    if world > 1:
        t = torch.tensor([total], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t.item())
    return total, per


# --------------------------------------------------------------------------------------
# CPU baseline (oracle port of the reference kernels)
# --------------------------------------------------------------------------------------
def cpu_sample(name, variant):
    """A bounded sample of the workload for the CPU oracle: whole requests / sequences with
    their full context and all heads, so that tokens per second of the sample is the rate of
    the workload.  Returns (run, tokens, description)."""
    from oracle import runner
    from lazy_attention_b200 import synth
    if name == "c4":
        case = synth.config_c4(device="cpu", variant=variant, batch=1, qlen=128)
        sample = ("1 of the 8 requests with its full context (128 x 512 cached tokens, all 32 heads) and 128 of "
                  "its 512 new tokens, one KV head after the other")
        op = "lazy_prefill" if variant == "lazy" else "mepic_prefill"
        run = lambda: runner.run_oracle_by_kv_head(case, op)  # noqa: E731
        tokens = 128
    elif name == "c3":
        case = synth.config_c3(device="cpu", variant=variant, batch=2)
        sample = "2 requests drawn as the workload's 32 are (20 documents each, all heads)"
        op = "lazy_prefill" if variant == "lazy" else "mepic_prefill"
        run = lambda: runner.run_oracle_by_kv_head(case, op)  # noqa: E731
        tokens = sum(case["q_lens"])
    elif name == "c2":
        case = synth.config_c2(device="cpu", variant=variant)
        sample = "the whole call"
        op = "lazy_prefill" if variant == "lazy" else "mepic_prefill"
        run = lambda: runner.run_oracle(case, op)  # noqa: E731
        tokens = 128
    else:
        docs, ks, vs = c5_documents(256)
        case = synth.build_decode(synth.GEOM_8B, torch.bfloat16, docs[:8], seed=0, device="cpu",
                                  kv_dtype="fp8_e4m3", variant=variant, k_scale=ks, v_scale=vs)
        sample = "the first 8 of the 256 sequences (all heads, full context)"
        op = "lazy_op" if variant == "lazy" else "mepic_op"
        run = lambda: runner.run_oracle(case, op)  # noqa: E731
        tokens = 8
    case["packed_block_table"] = runner.pack_host(case)
    return run, tokens, sample


def cpu_baseline(name, variant, budget_s=12.0):
    """Times the float32 torch oracle on the bounded sample with all host threads."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    run, tokens, sample = cpu_sample(name, variant)
    run()  # warm-up
    t0 = time.perf_counter()
    n = 0
    while True:
        run()
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 50:
            break
    dt = (time.perf_counter() - t0) / n
    return dict(value=tokens / dt, unit="tokens/s", cores=cores, kind="port",
                sample=f"{sample}; {n} calls of {dt:.2f} s")


def reference_arm(args):
    """K timed steps (after warm-up) of the CPU oracle, each step one call over the bounded
    sample; rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    run, tokens, sample = cpu_sample(args.workload, args.variant)
    for _ in range(max(1, min(args.warmup, 3))):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / args.steps
    winfo = workload_info(args.workload, int(os.environ.get("WORLD_SIZE", "1")), args.scale, args.kv_dtype)
    tok_s = tokens / dt
    line = dict(metric=METRIC, impl="reference", value=tok_s, unit="tokens/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 * dt, tokens_per_step=tokens, higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=winfo["workload"], variant=args.variant, kernel=args.kernel,
                            partition=winfo["partition"], l2=winfo["l2"]),
                cpu_baseline=dict(value=tok_s, unit="tokens/s", cores=cores, kind="port",
                                  sample=sample + "; each step is one call over this sample"),
                e2e=dict(value=tok_s, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# the reference's Triton kernels on this GPU (a baseline beside the timed regions, N = 1)
# --------------------------------------------------------------------------------------
def triton_baseline(case, info, ours_out, steps=3):
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        import triton_ref
        why = triton_ref.available()
        if why:
            return dict(unavailable=why)
        lazy = case["variant"] == "lazy"
        if info["kind"] == "prefill":
            op = "lazy_prefill" if lazy else "mepic_prefill"
        else:
            op = "lazy_op" if lazy else "mepic_op"
        out = torch.zeros_like(ours_out)
        t0 = time.perf_counter()
        triton_ref.run(case, op, out=out)          # compiles on first use
        torch.cuda.synchronize()
        first_s = time.perf_counter() - t0
        triton_ref.run(case, op, out=out)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for i in range(steps):
            triton_ref.run(case, op, out=out)
            ev[i + 1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[-1]) / steps
        diff = float((out.float() - ours_out.float()).abs().max().item())
        import triton
        return dict(ms_per_step=ms, steps=steps, first_call_s=first_s, max_abs_diff_vs_this_library=diff,
                    what="the reference's Triton operator with its own launch parameters, compiled by Triton "
                         f"{triton.__version__} for this GPU, same inputs, eager calls")
    except Exception as e:  # the baseline is optional: report why it is missing
        torch.cuda.synchronize()
        return dict(unavailable=f"{type(e).__name__}: {str(e)[:300]}")


# --------------------------------------------------------------------------------------
def run_workload(name, args, world, rank, local_rank, device):
    """Builds one workload on this rank, checks the gather (N > 1), times it device-resident
    and end to end, and returns the result fields (meaningful on rank 0)."""
    import torch.distributed as dist
    import lazy_attention_b200 as la
    from lazy_attention_b200 import sharding

    if world == 1 and args.shard_of > 1:
        case, info = build_workload(name, device, args.variant, 0, args.shard_of, args.scale, args.kv_dtype)
        info = dict(info, partition=f"rank 0's shard of {args.shard_of} ({info['partition']}), run alone")
    else:
        case, info = build_workload(name, device, args.variant, rank, world, args.scale, args.kv_dtype)
    flops, byts, units = algorithmic_work(case, info)
    step, out = make_step(case, info, args.kernel)
    g = case["geom"]
    steps, warmup = args.steps, args.warmup

    # ---- the job's totals.  A call sharded by KV-head group serves every token on every rank:
    # its tokens are counted once; FLOPs and bytes are partitioned and add up.
    tokens_all = units
    if world > 1 and info["partition"] == "request":
        t = torch.tensor([units], dtype=torch.float64, device=device)
        dist.all_reduce(t)
        tokens_all = int(t[0].item())

    def nccl_gather(o):
        if info["kind"] == "prefill":
            return sharding.gather_head_outputs(o, world)
        docs, _, _ = c5_documents(info["total_seqs"])
        rows = sharding.lpt_assign([sum(d) + 1 for d in docs], world)
        return sharding.gather_request_outputs(o, rows, info["total_seqs"])

    # ---- N > 1: how the ranks' results come together
    gather_mode, peers, gather_check = "none", None, None
    if world > 1 and args.gather == "fused":
        try:
            if info["kind"] == "prefill":
                mk = lambda: sharding.PeerOutput(case["num_tokens"], info["full_heads"][0], g.head_dim,  # noqa: E731
                                                 out.dtype, device, head_offset=rank * g.num_q_heads)
            else:
                mk = lambda: sharding.PeerOutput(info["total_seqs"], g.num_q_heads, g.head_dim, out.dtype,  # noqa: E731
                                                 device, row_map=case["global_rows"])
            peers = [mk(), mk()]  # two sets: a step's result is read while the next step is written
            gather_mode = "fused into the kernels (peer stores over NVLink) + " + (
                "signal kernel" if args.barrier == "signal" else "one-element all-reduce")
        except Exception as e:
            peers = None
            gather_mode = f"nccl all-gather (peer buffers unavailable: {type(e).__name__})"
    elif world > 1:
        gather_mode = "nccl all-gather"
    if peers is not None:
        # correctness gate: the rows the peers stored must equal, bit for bit, what the same
        # kernels write locally followed by an all-gather
        want = nccl_gather(step(peer_out=None).clone())
        ok = 1
        for pset in peers:
            pset.local.zero_()
            torch.cuda.synchronize(device)
            dist.barrier()
            step(peer_out=pset)
            pset.barrier(collective=True if args.barrier == "nccl" else None)
            torch.cuda.synchronize(device)
            ok &= int(torch.equal(pset.local, want))
        flag = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        gather_check = "bit-exact" if int(flag.item()) == 1 else "MISMATCH"
        if gather_check != "bit-exact":
            if rank == 0:
                print(json.dumps(dict(error=f"{name}: fused output gather differs from the all-gather")))
            raise SystemExit(3)

    # ---- one call's launches (attention kernel + split merge) captured once and replayed: the
    # Python wrapper's argument marshalling then costs nothing per step.  Collectives stay outside.
    launch_mode, launches_per_step = "eager", None

    def eager_step():
        return step(peer_out=peers[0] if peers else None)
    fast_step = eager_step
    if args.cuda_graph == "on":
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                for _ in range(2):
                    eager_step()
            torch.cuda.current_stream(device).wait_stream(side)
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            n0 = la.launch_count()
            with torch.cuda.graph(graph):
                eager_step()
            launches_per_step = la.launch_count() - n0

            def fast_step():
                graph.replay()
                return out
            launch_mode = "cuda graph replay"
        except Exception as e:  # capture unavailable: keep launching eagerly
            torch.cuda.synchronize(device)
            launch_mode = f"eager (graph capture failed: {type(e).__name__})"

    if peers is not None:
        def post(o, slot=0):
            peers[slot].barrier(collective=True if args.barrier == "nccl" else None)
            return peers[slot].local
    elif world > 1:
        def post(o, slot=0):
            return nccl_gather(o)
    else:
        def post(o, slot=0):
            return o

    def full_step(*a, slot=0, **kw):
        if a or kw:
            return post(step(*a, peer_out=peers[slot] if peers else None, **kw), slot)
        return post(fast_step(), 0)

    # ---- device-resident timing ---------------------------------------------------------
    flush = byts < 200e6
    launches0 = la.launch_count()
    with ClockSampler(local_rank) as clk:
        total_ms, per = time_steps(full_step, steps, warmup, device, world, flush)
    launches = la.launch_count() - launches0
    launches_timed = int(round(launches * steps / (steps + warmup)))
    if launches_per_step is not None:
        # the graph's kernels, plus the signal kernel that ends a step of the fused gather
        launches_timed = (launches_per_step + int(peers is not None and args.barrier == "signal")) * steps
    ms_per_step = total_ms / steps
    value = tokens_all / (ms_per_step * 1e-3)
    assert abs(value * ms_per_step * 1e-3 - tokens_all) < 1.0

    # ---- kernel-only time of this rank's attention call (roofline), replayed and eager ---------
    _, kper = time_steps(fast_step, steps, 1, device, 1, flush)
    kern_ms = sum(kper) / len(kper)
    _, eper = time_steps(eager_step, steps, warmup, device, 1, flush)
    eager_ms = sum(eper) / len(eper)
    pk = peaks()
    traffic = None
    if (world == 1 and args.scale == 1.0 and args.variant == "lazy" and args.kernel == "auto"
            and args.kv_dtype == "auto"):
        traffic = recorded_traffic(name)
    if info["kind"] == "prefill":
        achieved = flops / (kern_ms * 1e-3) / 1e12
        peak = pk["tf_burst"]
        roof = dict(bound="tensor", achieved=achieved, peak=peak, unit="TFLOP/s", frac=achieved / peak,
                    traffic=traffic, peak_kind="burst bf16 (cuBLAS), " + pk["src"],
                    frac_of_sustained_peak=achieved / pk["tf_sust"], frac_of_nominal_2250=achieved / 2250.0,
                    kernel_ms=kern_ms, algorithmic_flops=flops, algorithmic_bytes=byts)
    else:
        achieved = byts / (kern_ms * 1e-3) / 1e9
        roof = dict(bound="hbm", achieved=achieved, peak=pk["hbm"], unit="GB/s", frac=achieved / pk["hbm"],
                    traffic=traffic, peak_kind="copy bandwidth, " + pk["src"], frac_of_nominal_8000=achieved / 8000.0,
                    kernel_ms=kern_ms, algorithmic_flops=flops, algorithmic_bytes=byts)
    if world > 1:
        roof["scope"] = "rank 0's shard: its kernel time against its share of the work"
    # the whole job's work, spread evenly over the ranks, at the peak, against rank 0's kernel time
    work = torch.tensor([flops, byts], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(work)
    ideal_ms = (float(work[0]) / world / (roof["peak"] * 1e12) if roof["bound"] == "tensor"
                else float(work[1]) / world / (roof["peak"] * 1e9)) * 1e3
    roof["ideal_ms_per_rank_at_peak"] = ideal_ms
    speedup_vs_ideal = ideal_ms / kern_ms

    # ---- end to end through the public API with host buffers ----------------------------
    e2e = None
    if not args.no_e2e:
        hq, hk, hv = (case[n].cpu().pin_memory() for n in ("q", "k", "v"))
        tkeys = ["block_table", "q_offset", "q_mask", "query_start_loc", "seq_lens", "is_lazy"]
        if "packed_block_table" in case:
            tkeys.append("packed_block_table")
        htab = {n: case[n].cpu().pin_memory() for n in tkeys}
        dq, dk, dv = (torch.empty_like(case[n]) for n in ("q", "k", "v"))
        dtab = {n: torch.empty_like(case[n]) for n in tkeys}
        res = full_step()
        torch.cuda.synchronize(device)
        # the job reads the gathered result back once: rank r takes rows [r0, r1)
        r0, r1 = res.shape[0] * rank // world, res.shape[0] * (rank + 1) // world
        hout = torch.empty((r1 - r0,) + tuple(res.shape[1:]), dtype=res.dtype).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv)) + \
            sum(t.numel() * t.element_size() for t in htab.values())
        d2h = hout.numel() * hout.element_size()
        if world > 1:
            t = torch.tensor([h2d, d2h], dtype=torch.float64, device=device)
            dist.all_reduce(t)
            h2d, d2h = int(t[0].item()), int(t[1].item())

        def e2e_step():
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            for n in tkeys:
                dtab[n].copy_(htab[n], non_blocking=True)
            hout.copy_(full_step(dq, dk, dv, dtab)[r0:r1], non_blocking=True)

        e_total, _ = time_steps(e2e_step, steps, warmup, device, world, flush)
        serial_ms = e_total / steps

        # The same steps as a pipeline: two sets of device buffers, uploads on one stream, the
        # call on the current stream, the read-back on a third, so that a step's copies run
        # under its neighbours' attention call.  Every step still uploads its own inputs and
        # reads its own result back; the clock runs from before the first upload to after the
        # last read-back.
        cur = torch.cuda.current_stream(device)
        s_up, s_down = torch.cuda.Stream(device), torch.cuda.Stream(device)
        sets = []
        for _ in range(2):
            sets.append(dict(q=torch.empty_like(case["q"]), k=torch.empty_like(case["k"]),
                             v=torch.empty_like(case["v"]), tab={n: torch.empty_like(case[n]) for n in tkeys},
                             out=torch.empty_like(out), host=torch.empty_like(hout).pin_memory(),
                             up=torch.cuda.Event(), done=torch.cuda.Event(), down=torch.cuda.Event()))

        def pipelined(n_steps):
            for i in range(n_steps):
                b = sets[i % 2]
                with torch.cuda.stream(s_up):
                    s_up.wait_event(b["done"])       # the call that last read these inputs has finished
                    b["q"].copy_(hq, non_blocking=True)
                    b["k"].copy_(hk, non_blocking=True)
                    b["v"].copy_(hv, non_blocking=True)
                    for n in tkeys:
                        b["tab"][n].copy_(htab[n], non_blocking=True)
                    b["up"].record(s_up)
                cur.wait_event(b["up"])
                cur.wait_event(b["down"])            # the previous result in this buffer has been read back
                r = full_step(b["q"], b["k"], b["v"], b["tab"], out_=b["out"], slot=i % 2)
                b["done"].record(cur)
                with torch.cuda.stream(s_down):
                    s_down.wait_event(b["done"])
                    b["host"].copy_(r[r0:r1], non_blocking=True)
                    r.record_stream(s_down)
                    b["down"].record(s_down)
            for b in sets:
                cur.wait_event(b["down"])

        pipelined(warmup)
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(cur)
        s_up.wait_event(ev0)
        pipelined(steps)
        ev1.record(cur)
        torch.cuda.synchronize(device)
        p_total = ev0.elapsed_time(ev1)
        if world > 1:
            dist.barrier()
            tt = torch.tensor([p_total], dtype=torch.float64, device=device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            p_total = float(tt.item())
        piped_ms = p_total / steps
        best_ms = min(piped_ms, serial_ms)
        e2e = dict(value=tokens_all / (best_ms * 1e-3), unit="tokens/s",
                   h2d_bytes_per_step=int(h2d), d2h_bytes_per_step=int(d2h), ms_per_step=best_ms,
                   serial_ms_per_step=serial_ms, pipelined_ms_per_step=piped_ms,
                   mode="uploads and read-backs pipelined under the neighbouring steps' calls"
                   if piped_ms <= serial_ms else "upload, call and read-back in sequence on one stream")

    res = dict(value=value, unit="tokens/s", ms_per_step=ms_per_step, tokens_per_step=tokens_all,
               scaling=info["scaling"],
               dtype="bf16" if info["kind"] == "prefill" and "fp8" not in args.kv_dtype else
               f"bf16 query, {case['kv_cache_dtype'].replace('auto', 'bf16').replace('fp8_', '')} KV, f32 accumulate",
               config=dict(workload=info["workload"], variant=args.variant, kernel=args.kernel,
                           partition=info["partition"], l2=info["l2"]),
               execution=dict(launch=launch_mode, gather=gather_mode, eager_ms_per_step=eager_ms,
                              replay_ms_per_step=kern_ms),
               roofline=roof, speedup_vs_ideal=speedup_vs_ideal, e2e=e2e, gpu_launches=launches_timed,
               clocks=clk.summary())
    if gather_check is not None:
        res["gather_check"] = gather_check
    if world == 1 and not args.no_triton and args.scale == 1.0 and args.shard_of == 1:
        tb = triton_baseline(case, info, fast_step())
        if "ms_per_step" in tb:
            tb["value"] = tokens_all / (tb["ms_per_step"] * 1e-3)
            tb["unit"] = "tokens/s"
            res["speedup_vs_triton"] = tb["ms_per_step"] / eager_ms
        res["triton_baseline"] = tb
    if peers is not None:
        torch.cuda.synchronize(device)
        for pset in peers:
            pset.close()
    return res


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the library has no CPU path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    head = run_workload(args.workload, args, world, rank, local_rank, device)
    torch.cuda.empty_cache()
    also = {}
    if not args.no_also and args.scale == 1.0 and args.workload == "c4" and args.kv_dtype == "auto" \
            and args.shard_of == 1:
        for name in ["c5"] + (["c3", "c2"] if world == 1 else []):
            r = run_workload(name, args, world, rank, local_rank, device)
            torch.cuda.empty_cache()
            also[name] = {k: r[k] for k in ("value", "unit", "ms_per_step", "tokens_per_step", "dtype", "config",
                                            "execution", "roofline", "speedup_vs_ideal", "e2e", "gpu_launches", "gather_check",
                                            "triton_baseline", "speedup_vs_triton") if k in r}

    if rank == 0:
        line = dict(metric=METRIC, value=head["value"], unit="tokens/s", n_gpus=world, steps=args.steps,
                    warmup=args.warmup, ms_per_step=head["ms_per_step"], higher_is_better=True,
                    scaling=head["scaling"], vs_baseline=None, dtype=head["dtype"], data="synthetic",
                    tokens_per_step=head["tokens_per_step"], config=head["config"], execution=head["execution"],
                    roofline=head["roofline"], speedup_vs_ideal=head["speedup_vs_ideal"], e2e=head["e2e"],
                    gpu_launches=head["gpu_launches"] + sum(a["gpu_launches"] for a in also.values()),
                    clocks=head["clocks"])
        for k in ("gather_check", "triton_baseline", "speedup_vs_triton"):
            if k in head:
                line[k] = head[k]
        if also:
            line["also"] = also
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(args.workload, args.variant)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
