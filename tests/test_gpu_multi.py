"""Two-GPU check of the output gather fused into the kernels' epilogue: the
result rows stored straight into every rank's buffer must equal, bit for bit,
what the same kernels write locally followed by an all-gather.  Skipped on
boxes with fewer than two GPUs (the sharding logic itself is covered on CPU
ranks in test_sharding.py)."""
import os
import sys
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import torch.distributed as dist
    import lazy_attention_b200 as la
    from lazy_attention_b200 import sharding, synth
    import util
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=device)
    try:
        # ---- prefill sharded by KV-head group
        pool = [512, 256, 1024, 160]
        reqs = [dict(docs=[0, 2, 1], qlen=300), dict(docs=[3, 0], qlen=77), dict(docs=[1], qlen=512)]
        full = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, pool, reqs, seed=21, device=device)
        mine = sharding.shard_by_kv_head(full, rank, world)
        g = mine["geom"]

        def run(peer):
            o = torch.zeros(mine["num_tokens"], g.num_q_heads, g.head_dim, dtype=torch.bfloat16, device=device)
            la.context_attention_fwd(mine["q"], mine["k"], mine["v"], o, mine["kv_cache_dtype"], mine["k_cache"],
                                     mine["v_cache"], mine["block_table"], mine["query_start_loc"], mine["seq_lens"],
                                     mine["max_seq_len"], mine["max_query_len"], mine["k_scale"], mine["v_scale"],
                                     sm_scale=mine["sm_scale"], cos_sin_cache=mine["cos_sin_cache"],
                                     is_lazy=mine["is_lazy"], q_offset=mine["q_offset"], q_mask=mine["q_mask"],
                                     kernel="tensor", peer_out=peer)
            return o
        peer = sharding.PeerOutput(mine["num_tokens"], full["geom"].num_q_heads, g.head_dim, torch.bfloat16, device,
                                   head_offset=rank * g.num_q_heads)
        ok_prefill = True
        # one split: the attention kernel's epilogue stores the rows; three: the merge kernel.
        # The ranks reach each barrier at different times (host-side delays of different
        # lengths), and a rank clears its buffer between two barriers, so a barrier that lets
        # a rank through early shows up as missing rows.
        for it, splits in enumerate(["1", "3", "1", "3"]):
            os.environ["LAZY_ATTN_B200_PREFILL_SPLITS"] = splits
            want = sharding.gather_head_outputs(run(None), world)
            peer.local.zero_()
            time.sleep(0.03 * ((rank + it) % world))
            peer.barrier()
            run(peer)
            time.sleep(0.02 * ((rank + it + 1) % world))
            peer.barrier()
            torch.cuda.synchronize(device)
            ok_prefill = ok_prefill and bool(torch.equal(peer.local, want))
        os.environ.pop("LAZY_ATTN_B200_PREFILL_SPLITS", None)
        # ---- decode sharded by request
        dec = synth.build_decode(synth.GEOM_8B, torch.bfloat16, [[512, 1024], [256], [2048, 160], [512], [1024, 1024]],
                                 seed=22, device=device, kv_dtype="fp8_e4m3", k_scale=0.1, v_scale=0.2)
        dec["packed_block_table"] = util.pack_host(dec).to(device)
        part = sharding.shard_by_request(dec, rank, world)
        gd = dec["geom"]

        def run_dec(peer):
            o = torch.zeros(part["num_tokens"], gd.num_q_heads, gd.head_dim, dtype=torch.bfloat16, device=device)
            la.chunked_prefill_paged_decode(part["q"], part["k"], part["v"], o, part["kv_cache_dtype"], part["k_cache"],
                                            part["v_cache"], part["block_table"], part["query_start_loc"],
                                            part["seq_lens"], part["max_seq_len"], 1, part["k_scale"], part["v_scale"],
                                            sm_scale=part["sm_scale"], cos_sin_cache=part["cos_sin_cache"],
                                            is_lazy=part["is_lazy"], q_offset=part["q_offset"], q_mask=part["q_mask"],
                                            packed_block_table=part["packed_block_table"], kernel="tensor",
                                            peer_out=peer)
            return o
        rows = [None] * world
        dist.all_gather_object(rows, part["request_rows"])
        want_d = sharding.gather_request_outputs(run_dec(None), rows, dec["num_tokens"])
        peer_d = sharding.PeerOutput(dec["num_tokens"], gd.num_q_heads, gd.head_dim, torch.bfloat16, device,
                                     row_map=part["request_rows"])
        run_dec(peer_d)
        peer_d.barrier()
        torch.cuda.synchronize(device)
        ok_decode = bool(torch.equal(peer_d.local, want_d))
        status = la.device_status()
        q.put((rank, ok_prefill, ok_decode, status))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_gather_equals_all_gather():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=_worker, args=(r, world, 29533, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.kill()
    results = sorted(q.get(timeout=10) for _ in range(world))
    for rank, ok_prefill, ok_decode, status in results:
        assert status == 0, f"rank {rank}: device status {status}"
        assert ok_prefill, f"rank {rank}: prefill rows stored by the peers differ from the all-gather"
        assert ok_decode, f"rank {rank}: decode rows stored by the peers differ from the all-gather"
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensors_on_a_device_that_is_not_current():
    """One process, tensors on cuda:1 while cuda:0 is current: the operators launch on the
    tensors' device and stream (tensor maps, status word, kernel attributes are per device)."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import lazy_attention_b200 as la
    from lazy_attention_b200 import synth
    import util
    assert torch.cuda.current_device() == 0
    pool = [100, 64, 33, 250, 16, 129]
    reqs = [dict(docs=[2, 0, 1], qlen=37), dict(docs=[3, 1, 5], qlen=300), dict(docs=[1, 2, 4], qlen=1)]
    for dev in ("cuda:1", "cuda:0", "cuda:1"):
        case = synth.build_prefill(synth.GEOM_8B, torch.bfloat16, pool, reqs, seed=7, variant="lazy", device=dev)
        case["packed_block_table"] = util.pack_host(case).to(dev)
        out = util.new_out(case)
        la.chunked_prefill_paged_decode(
            case["q"], case["k"], case["v"], out, case["kv_cache_dtype"], case["k_cache"], case["v_cache"],
            case["block_table"], case["query_start_loc"], case["seq_lens"], case["max_seq_len"], case["max_query_len"],
            case["k_scale"], case["v_scale"], sm_scale=case["sm_scale"], cos_sin_cache=case["cos_sin_cache"],
            is_lazy=case["is_lazy"], q_offset=case["q_offset"], q_mask=case["q_mask"],
            packed_block_table=case["packed_block_table"], kernel="tensor")
        torch.cuda.synchronize(dev)
        assert torch.cuda.current_device() == 0
        with torch.cuda.device(dev):
            assert la.device_status() == 0
        util.assert_close(out.float().cpu(), util.run_oracle(case, "lazy_op"), atol=2e-2, rtol=1e-2, what=f"on {dev}")
