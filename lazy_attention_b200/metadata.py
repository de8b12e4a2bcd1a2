"""Rotation metadata: what the scheduler emits per request and how the model
runner packs it for the kernels.  Integer work, bit-exact with the reference.

* ``metadata_for_lazy_attention`` / ``metadata_for_mepic`` /
  ``metadata_for_variant``: lazy_attn/lazy/core/sched/scheduler.py:758-794
* ``max_rotation_offset`` / ``MAX_PACKED_Q_OFFSET``: lazy_attn/lazy/utils/rotation.py:15-37
* ``validate_rotation_offsets``: lazy_attn/lazy/engine/processor.py:128-148
* ``LazyMetadataBuffers`` / ``pack_block_table``:
  lazy_attn/lazy/worker/gpu_model_runner.py:91-153,193-239,296-343
"""
from __future__ import annotations

import os
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib

MAX_PACKED_Q_OFFSET = 0xFFFF


def _lens(request_or_lens, padded=None):
    if padded is None:
        return list(request_or_lens.document_lens), list(request_or_lens.document_lens_padded)
    return list(request_or_lens), list(padded)


def metadata_for_lazy_attention(request, block_size_or_padded, block_size: Optional[int] = None
                                ) -> Tuple[List[int], List[int]]:
    """Per-page ``q_offset`` (+1-biased rotation position) and ``q_mask`` (pad
    count on a document's last page) for the documents of a request, plus one
    trailing entry (offset 1, mask 0) for the query page.

    Call as ``metadata_for_lazy_attention(request, block_size)`` with an object
    carrying ``document_lens`` / ``document_lens_padded`` (the reference's
    signature) or as ``metadata_for_lazy_attention(lens, lens_padded, block_size)``.
    """
    if block_size is None:
        lens, padded = _lens(request)
        bs = int(block_size_or_padded)
    else:
        lens, padded = _lens(request, block_size_or_padded)
        bs = int(block_size)
    n_blocks = sum(padded) // bs + 1
    q_mask = np.zeros(n_blocks, dtype=np.int32)
    q_offset = np.zeros(n_blocks, dtype=np.int32)
    pads = np.asarray(padded, dtype=np.int64) - np.asarray(lens, dtype=np.int64)
    position = int(pads.sum()) if len(lens) else 0
    cursor = 0
    for true_len, padded_len, pad in zip(lens, padded, pads):
        n = padded_len // bs
        q_offset[cursor:cursor + n] = position + 1
        cursor += n
        q_mask[cursor - 1] = pad
        position += true_len
    q_offset[cursor] = 1
    return [int(v) for v in q_offset], [int(v) for v in q_mask]


def metadata_for_mepic(request, block_size_or_padded, block_size: Optional[int] = None):
    """Per-token variant: no offsets, same pad mask."""
    q_offset, q_mask = metadata_for_lazy_attention(request, block_size_or_padded, block_size)
    return [0] * len(q_offset), q_mask


def metadata_for_variant(request, block_size_or_padded, block_size: Optional[int] = None):
    """Selects by ``LAZY_ATTENTION_VARIANT`` as the reference does
    (lazy_attn/lazy/utils/variants.py:53-86): ``mepic`` / ``nope`` /
    ``position_independent`` or the default ``lazy``."""
    name = "lazy"
    for key in ("LAZY_ATTENTION_VARIANT", "LAZY_ATTENTION_MODE", "VLLM_LAZY_VARIANT"):
        if os.environ.get(key):
            name = os.environ[key].strip().lower()
            break
    if name in ("mepic", "nope", "position_independent"):
        return metadata_for_mepic(request, block_size_or_padded, block_size)
    return metadata_for_lazy_attention(request, block_size_or_padded, block_size)


def max_rotation_offset(document_lens: Sequence[int], document_lens_padded: Sequence[int]) -> int:
    """Largest ``q_offset`` the metadata will hold: total padding plus the true
    lengths of all documents but the last, plus one."""
    if not document_lens:
        return 0
    pad = sum(p - t for t, p in zip(document_lens, document_lens_padded))
    return pad + sum(document_lens[:-1]) + 1


def validate_rotation_offsets(document_lens, document_lens_padded) -> None:
    """Admission check: refuse a request whose offsets do not fit 16 bits."""
    worst = max_rotation_offset(document_lens, document_lens_padded)
    if worst > MAX_PACKED_Q_OFFSET:
        raise ValueError(
            f"documents need a rotation offset of {worst}, past the "
            f"{MAX_PACKED_Q_OFFSET} the packed block table's 16-bit field holds")


def pack_block_table(block_table: torch.Tensor, q_offset: torch.Tensor, q_mask: torch.Tensor,
                     out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                     num_rows: Optional[int] = None) -> torch.Tensor:
    """``out[r, c] = block << 32 | q_offset << 16 | q_mask`` in one CUDA launch.

    ``rows`` (int32 device tensor) restricts the rebuild to those rows (the
    reference's delta rebuild); otherwise rows ``0 .. num_rows-1`` are written.
    """
    if not block_table.is_cuda:
        raise RuntimeError("pack_block_table runs on CUDA tensors only")
    for t in (block_table, q_offset, q_mask):
        if t.dtype != torch.int32 or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError("block_table / q_offset / q_mask must be 2-D int32 with unit inner stride")
    n_cols = block_table.shape[1]
    if q_offset.shape[1] < n_cols or q_mask.shape[1] < n_cols:
        raise ValueError("q_offset / q_mask have fewer columns than the block table")
    if not (block_table.stride(0) == q_offset.stride(0) == q_mask.stride(0)):
        raise ValueError("block_table, q_offset and q_mask must share one row stride")
    if out is None:
        out = torch.zeros(block_table.shape, dtype=torch.int64, device=block_table.device)
    if out.dtype != torch.int64 or out.stride(1) != 1 or out.shape[1] < n_cols:
        raise ValueError("out must be int64 with unit inner stride and enough columns")
    if rows is not None:
        if rows.dtype != torch.int32 or not rows.is_cuda:
            raise ValueError("rows must be an int32 CUDA tensor")
        n_rows, rows_ptr = rows.numel(), rows.data_ptr()
    else:
        n_rows = block_table.shape[0] if num_rows is None else int(num_rows)
        rows_ptr = None
    lib = _lib.load()
    with torch.cuda.device(block_table.device):
        rc = lib.la_pack_block_table(block_table.data_ptr(), q_offset.data_ptr(), q_mask.data_ptr(),
                                     out.data_ptr(), rows_ptr, n_rows, n_cols,
                                     block_table.stride(0), out.stride(0),
                                     torch.cuda.current_stream(block_table.device).cuda_stream)
    _lib.check(rc, "la_pack_block_table")
    return out


class LazyMetadataBuffers:
    """Persistent per-request rotation buffers and packed block tables, one table
    per KV-cache group (block ids are only meaningful inside their group).

    Mirrors the state ``LazyGPUModelRunner`` keeps: ``is_lazy`` / ``lazy_variant``
    ``[max_reqs]``, ``lazy_offset`` / ``lazy_mask`` ``[max_reqs, max_blocks]``
    with pinned host twins, a full rebuild after any batch change and a row-wise
    rebuild when only some rows grew.
    """

    def __init__(self, max_num_reqs: int, max_num_blocks_per_req: int, device="cuda",
                 num_kv_groups: int = 1, pin_memory: Optional[bool] = None):
        dev = torch.device(device)
        if pin_memory is None:
            pin_memory = dev.type == "cuda"
        self.device = dev
        self.max_num_reqs = max_num_reqs
        self.max_num_blocks_per_req = max_num_blocks_per_req

        def pair(shape, dtype):
            host = torch.zeros(shape, dtype=dtype, pin_memory=pin_memory)
            return host, torch.zeros(shape, dtype=dtype, device=dev)

        self.is_lazy_req_cpu, self.is_lazy_req = pair((max_num_reqs, ), torch.bool)
        self.lazy_variant_cpu, self.lazy_variant = pair((max_num_reqs, ), torch.int32)
        shape2 = (max_num_reqs, max_num_blocks_per_req)
        self.lazy_offset_cpu, self.lazy_offset = pair(shape2, torch.int32)
        self.lazy_mask_cpu, self.lazy_mask = pair(shape2, torch.int32)
        self.lazy_offset_np = self.lazy_offset_cpu.numpy()
        self.lazy_mask_np = self.lazy_mask_cpu.numpy()
        self.lazy_variant_np = self.lazy_variant_cpu.numpy()
        self.packed_block_tables = [torch.zeros(shape2, dtype=torch.int64, device=dev)
                                    for _ in range(num_kv_groups)]
        self.full_rebuild = True
        self.delta_rows: set = set()

    def refresh(self, requests: Iterable) -> None:
        """Copy each request's ``is_lazy, lazy_variant, q_offset, q_mask`` into
        the buffers (row = position in ``requests``) and upload them.  Refuses an
        offset past ``MAX_PACKED_Q_OFFSET`` rather than corrupting the block id."""
        requests = list(requests)
        n = len(requests)
        self.is_lazy_req_cpu[:n].fill_(False)
        self.lazy_variant_cpu[:n].fill_(0)
        self.lazy_offset_cpu[:n].fill_(0)
        self.lazy_mask_cpu[:n].fill_(0)
        any_lazy = False
        for idx, req in enumerate(requests):
            if not getattr(req, "is_lazy", False):
                continue
            any_lazy = True
            self.is_lazy_req_cpu[idx] = True
            self.lazy_variant_np[idx] = getattr(req, "lazy_variant", 0)
            q_offset = getattr(req, "q_offset", None)
            q_mask = getattr(req, "q_mask", None)
            if q_offset is not None:
                if len(q_offset) and max(q_offset) > MAX_PACKED_Q_OFFSET:
                    raise ValueError(
                        f"request {getattr(req, 'req_id', idx)}: q_offset {max(q_offset)} does not fit the "
                        f"16 bits the packed block table gives it (limit {MAX_PACKED_Q_OFFSET}); packing it "
                        f"would overwrite the block id, so the request must be rejected before it is scheduled")
                self.lazy_offset_np[idx, :len(q_offset)] = q_offset
            if q_mask is not None:
                self.lazy_mask_np[idx, :len(q_mask)] = q_mask
        self.is_lazy_req[:n].copy_(self.is_lazy_req_cpu[:n], non_blocking=True)
        self.lazy_variant[:n].copy_(self.lazy_variant_cpu[:n], non_blocking=True)
        if any_lazy:
            self.lazy_offset[:n].copy_(self.lazy_offset_cpu[:n], non_blocking=True)
            self.lazy_mask[:n].copy_(self.lazy_mask_cpu[:n], non_blocking=True)
        self.full_rebuild = True
        self.delta_rows.clear()

    def mark_rows_changed(self, rows: Iterable[int]) -> None:
        self.delta_rows.update(int(r) for r in rows)

    def rebuild_packed_block_table(self, block_tables: Sequence[torch.Tensor], num_reqs: int) -> int:
        """Refresh the packed tables from the per-group device block tables.
        Returns the number of rows rewritten per group."""
        if not (self.full_rebuild or self.delta_rows):
            return 0
        rows_t = None
        if not self.full_rebuild:
            rows = sorted(r for r in self.delta_rows if r < num_reqs)
            if not rows:
                self.delta_rows.clear()
                return 0
            rows_t = torch.tensor(rows, dtype=torch.int32, device=self.device)
        for table, packed in zip(block_tables, self.packed_block_tables):
            if table.shape[1] != packed.shape[1] or table.stride(0) != self.lazy_offset.stride(0):
                raise ValueError("a group's block table must have the shape and row stride "
                                 "of the rotation buffers [max_reqs, max_blocks]")
            pack_block_table(table, self.lazy_offset, self.lazy_mask, out=packed, rows=rows_t,
                             num_rows=num_reqs)
        n = num_reqs if self.full_rebuild else rows_t.numel()
        self.full_rebuild = False
        self.delta_rows.clear()
        return n

    def attach(self, metadata, num_reqs: int, group_idx: int = 0):
        """Attach the rotation tensors to an attention-metadata object, as
        ``_attach_lazy_attn_metadata`` does."""
        metadata.is_lazy = self.is_lazy_req[:num_reqs]
        metadata.lazy_variant = self.lazy_variant[:num_reqs]
        metadata.q_offset = self.lazy_offset[:num_reqs]
        metadata.q_mask = self.lazy_mask[:num_reqs]
        metadata.packed_block_table = self.packed_block_tables[group_idx][:num_reqs]
        return metadata
