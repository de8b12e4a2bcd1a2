"""Multi-GPU partitioning of the attention call.

Attention is independent per (request, KV head), so the call shards without any
data-path exchange; only the outputs are gathered at the end.

* :func:`shard_by_kv_head` -- rank ``r`` of ``g`` owns KV heads
  ``[r*Hkv/g, (r+1)*Hkv/g)`` and the query heads of those groups (what tensor
  parallelism gives each rank); tables and the cos/sin table are replicated.
* :func:`shard_by_request` -- rank ``r`` owns a subset of the sequences, chosen
  by longest-processing-time-first on the context length so that ranks get
  equal work, with all heads.
* :func:`gather_head_outputs` / :func:`gather_request_outputs` -- one
  all-gather of the per-rank outputs (NCCL on GPUs, gloo in the CPU tests).

The reference has no multi-GPU path of its own (its data-parallel engine class
is an empty stub, lazy_attn/lazy/engine/core.py:154-156).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import torch


def head_range(num_kv_heads: int, rank: int, world: int):
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} KV heads do not split over {world} ranks")
    per = num_kv_heads // world
    return rank * per, (rank + 1) * per


def shard_by_kv_head(case: Dict, rank: int, world: int) -> Dict:
    """Slice a call built for all heads down to this rank's KV-head group."""
    geom = case["geom"]
    lo, hi = head_range(geom.num_kv_heads, rank, world)
    G = geom.num_q_heads // geom.num_kv_heads
    out = dict(case)
    out["q"] = case["q"][:, lo * G:hi * G]
    out["k"] = case["k"][:, lo:hi]
    out["v"] = case["v"][:, lo:hi]
    out["k_cache"] = case["k_cache"][:, lo:hi]
    out["v_cache"] = case["v_cache"][:, lo:hi]
    out["geom"] = type(geom)(geom.num_q_heads // world, geom.num_kv_heads // world,
                             geom.head_dim, geom.block_size, geom.rope_theta)
    out["head_slice"] = (lo * G, hi * G)
    return out


def lpt_assign(costs: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time-first: items sorted by decreasing cost, each given
    to the currently lightest rank.  Deterministic; every rank computes the same."""
    order = sorted(range(len(costs)), key=lambda i: (-int(costs[i]), i))
    loads = [0] * world
    bins: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (loads[j], j))
        bins[r].append(i)
        loads[r] += int(costs[i])
    return [sorted(b) for b in bins]


def shard_by_request(case: Dict, rank: int, world: int) -> Dict:
    """Keep only this rank's sequences of a decode call (one query token each)."""
    seq_lens = case["seq_lens"].cpu().tolist()
    mine = lpt_assign(seq_lens, world)[rank]
    idx = torch.tensor(mine, dtype=torch.long, device=case["q"].device)
    out = dict(case)
    n = len(mine)
    qsl = case["query_start_loc"].cpu().tolist()
    rows = torch.tensor([qsl[i] for i in mine], dtype=torch.long, device=case["q"].device)
    q = case["q"][rows]
    out["q"] = torch.cat([q, q[:1]], dim=0) if n else q  # one row of slack, as the caller passes
    out["k"] = case["k"][rows]
    out["v"] = case["v"][rows]
    for key in ("block_table", "q_offset", "q_mask", "packed_block_table"):
        if key in case and case[key] is not None:
            out[key] = case[key][idx].contiguous()
    out["is_lazy"] = case["is_lazy"][idx]
    out["seq_lens"] = case["seq_lens"][idx].contiguous()
    out["query_start_loc"] = torch.arange(n + 1, dtype=torch.int32, device=case["q"].device)
    out["num_tokens"] = n
    out["max_seq_len"] = max([seq_lens[i] for i in mine], default=0)
    out["request_rows"] = [qsl[i] for i in mine]
    return out


def gather_head_outputs(local_out: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """All-gather ``[T, Hq/world, D]`` outputs into ``[T, Hq, D]`` (rank-major heads)."""
    import torch.distributed as dist
    if world == 1:
        return local_out
    T, h, d = local_out.shape
    gathered = torch.empty((world * T, h, d), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(gathered, local_out.contiguous(), group=group)
    return gathered.view(world, T, h, d).permute(1, 0, 2, 3).reshape(T, world * h, d)


def gather_request_outputs(local_out: torch.Tensor, rows_per_rank: Sequence[Sequence[int]],
                           total_rows: int, group=None) -> torch.Tensor:
    """All-gather per-rank ``[n_r, Hq, D]`` outputs (padded to the largest share)
    and scatter them back to their original rows."""
    import torch.distributed as dist
    world = len(rows_per_rank)
    if world == 1:
        return local_out
    cap = max(len(r) for r in rows_per_rank)
    _, h, d = local_out.shape
    padded = torch.zeros((cap, h, d), dtype=local_out.dtype, device=local_out.device)
    padded[:local_out.shape[0]] = local_out
    gathered = torch.empty((world * cap, h, d), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(gathered, padded, group=group)
    gathered = gathered.view(world, cap, h, d)
    full = torch.zeros((total_rows, h, d), dtype=local_out.dtype, device=local_out.device)
    for r, rows in enumerate(rows_per_rank):
        if rows:
            full[torch.tensor(rows, dtype=torch.long, device=full.device)] = gathered[r, :len(rows)]
    return full


class _DeviceView:
    """Exposes raw device memory to torch through the CUDA array interface (16-bit words)."""

    def __init__(self, ptr: int, words: int):
        self.__cuda_array_interface__ = dict(shape=(words,), typestr="<i2", data=(int(ptr), False), version=3)


def _as_tensor(ptr: int, shape, dtype, device) -> torch.Tensor:
    n = 1
    for d in shape:
        n *= int(d)
    if torch.empty((), dtype=dtype).element_size() != 2:
        raise ValueError("peer output buffers hold 16-bit elements (bf16 / fp16)")
    return torch.as_tensor(_DeviceView(ptr, n), device=device).view(dtype).view(*shape)


class PeerOutput:
    """Full-size output buffers of all ranks of one node, each mapped into every
    rank's process, for the gather fused into the kernels' epilogue.

    Every rank allocates ``[rows, heads, head_dim]`` through the library
    (``la_peer_alloc``), exports it with CUDA IPC (``la_peer_export``) and opens the
    others' (``la_peer_open``); the attention kernels then store each result row straight
    into all of these buffers (``peer_out=`` of the operators), and
    :meth:`barrier` is all that remains of the collective: one small kernel on the
    current stream (``la_peer_barrier``) in which every rank announces, with a store
    into each peer's signal buffer, that its kernels of the step have finished, and
    waits (bounded) for the others' announcements.  Ranks that share a GPU fall back
    to a one-element all-reduce: their kernels must not wait on one another on one
    device.  ``head_offset`` is the position of this
    rank's first head in the full buffers (KV-head sharding); ``rows`` maps local
    output rows to rows of the full buffers (request sharding).

    The buffers are rewritten by the peers' next call: read :attr:`local` (or
    copy it) before the ranks pass the next barrier, or alternate two instances.
    Call :meth:`close` (all ranks) to unmap and free them.
    """

    def __init__(self, rows: int, heads: int, head_dim: int, dtype, device, head_offset: int = 0,
                 row_map=None, group=None):
        import ctypes as C
        import torch.distributed as dist
        from . import _lib
        lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        shape = (rows, heads, head_dim)
        nbytes = rows * heads * head_dim * 2
        self._lib, self._own, self._mapped = lib, None, []
        self._own_signal, self._signals, self._signal_array = None, [], None
        # Every rank runs the same collectives whatever happens locally, and all
        # ranks fail together if any of them could not export or map a buffer.
        ok, handle = 1, None

        def alloc_and_export(size):
            own = C.c_void_p()
            if lib.la_peer_alloc(size, C.byref(own)) != 0:
                return None, None
            buf = C.create_string_buffer(64)
            if lib.la_peer_export(own.value, buf) != 0:
                return own.value, None
            return own.value, buf.raw

        def open_peer(h):
            # opened with THIS rank's GPU current: the mapping is made for the GPU whose
            # kernels will store through it
            mapped = C.c_void_p()
            if h is None or lib.la_peer_open(h, C.byref(mapped)) != 0:
                return None
            self._mapped.append(mapped.value)
            return mapped.value

        with torch.cuda.device(device):
            self._own, handle = alloc_and_export(nbytes)
            self._own_signal, signal_handle = alloc_and_export(_lib.LA_PEER_SIGNAL_BYTES)
            if handle is None or signal_handle is None:
                ok = 0
            gpu = str(torch.cuda.get_device_properties(device).uuid)
            handles = [None] * self.world
            dist.all_gather_object(handles, (handle, signal_handle, gpu), group=group)
            self.buffers = []
            for r, (h, hs, _) in enumerate(handles):
                if r == self.rank and self._own is not None and self._own_signal is not None:
                    self.buffers.append(_as_tensor(self._own, shape, dtype, device))
                    self._signals.append(self._own_signal)
                    continue
                ptr, sig = open_peer(h), open_peer(hs)
                if ptr is None or sig is None:
                    ok = 0
                    continue
                self.buffers.append(_as_tensor(ptr, shape, dtype, device))
                self._signals.append(sig)
            gpus = [g for (_, _, g) in handles]
            self._one_rank_per_gpu = len(set(gpus)) == len(gpus)
            torch.cuda.synchronize(device)
        flag = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            self.close(collective=False)
            raise RuntimeError("peer-mapped output buffers are unavailable on at least one rank: " + _lib.last_error())
        self.local = self.buffers[self.rank]
        self.head_offset = int(head_offset)
        self.rows = None
        if row_map is not None:
            self.rows = torch.as_tensor(list(row_map), dtype=torch.int32).to(device)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        self._device = device
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def fill(self, peer) -> None:
        """Writes this object into a ``LaPeerOut`` of the C ABI."""
        for r, t in enumerate(self.buffers):
            peer.out[r] = t.data_ptr()
        peer.num_peers = self.world
        peer.head_offset = self.head_offset
        peer.stride_t, peer.stride_h = self.local.stride(0), self.local.stride(1)
        peer.rows = self.rows.data_ptr() if self.rows is not None else None

    def barrier(self, collective: Optional[bool] = None) -> None:
        """All ranks' kernels of the current step have finished and their rows have landed
        (stream-ordered).  ``collective=True`` uses a one-element all-reduce instead of the
        library's signal kernel (the default only for ranks that share a GPU)."""
        import torch.distributed as dist
        if collective is None:
            collective = not self._one_rank_per_gpu
        elif not collective and not self._one_rank_per_gpu:
            raise RuntimeError("ranks that share a GPU cannot wait for one another inside kernels")
        if collective:
            dist.all_reduce(self._flag, group=self.group)
            return
        if self._signal_array is None:
            self._signal_array = (ctypes.c_void_p * self.world)(*self._signals)
        stream = torch.cuda.current_stream(self._device).cuda_stream
        if torch.cuda.current_device() == self._device.index:
            code = self._lib.la_peer_barrier(self._signal_array, self.world, self.rank, stream)
        else:
            with torch.cuda.device(self._device):
                code = self._lib.la_peer_barrier(self._signal_array, self.world, self.rank, stream)
        if code != 0:
            from . import _lib
            raise RuntimeError(_lib.last_error())

    def close(self, collective: bool = True) -> None:
        """Unmaps the peers' buffers, then (after a barrier, so that no peer still has this
        rank's buffer mapped) frees this rank's own.  Tensors taken from :attr:`buffers`
        must not be used afterwards."""
        import torch.distributed as dist
        self.buffers = []
        self.local = None
        self._signals, self._signal_array = [], None
        for ptr in self._mapped:
            self._lib.la_peer_close(ptr)
        self._mapped = []
        if collective:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        for name in ("_own", "_own_signal"):
            if getattr(self, name) is not None:
                self._lib.la_peer_free(getattr(self, name))
                setattr(self, name, None)
