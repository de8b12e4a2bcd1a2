"""lazy_attention_b200: deferred-RoPE paged prefix-prefill and decode attention
for NVIDIA B200 (sm_100a), behind the operator surface of the reference's
``lazy_attn`` attention backend.

Public API (same names and argument meaning as the reference):

* :func:`context_attention_fwd`, :func:`chunked_prefill_paged_decode` -- the
  per-page ("lazy") variant;
* :func:`context_attention_fwd_mepic`, :func:`chunked_prefill_paged_decode_mepic`
  -- the per-token ("mepic") variant;
* :func:`metadata_for_lazy_attention`, :func:`metadata_for_mepic`,
  :func:`max_rotation_offset`, :class:`LazyMetadataBuffers`,
  :func:`pack_block_table` -- the scheduler / model-runner integer side;
* :func:`build_cos_sin_table` -- the cos/sin table builder.

All compute runs in ``liblazy_attention_b200.so`` (hand-written CUDA); there is
no CPU path.
"""
from .metadata import (MAX_PACKED_Q_OFFSET, LazyMetadataBuffers,
                       max_rotation_offset, metadata_for_lazy_attention,
                       metadata_for_mepic, metadata_for_variant,
                       pack_block_table, validate_rotation_offsets)
from .rope import ROPE_DEFAULT, ROPE_LLAMA3, build_cos_sin_table, rope_meta_from_layer
from .cache import write_to_paged_cache
from .attention import (chunked_prefill_paged_decode,
                        chunked_prefill_paged_decode_mepic,
                        context_attention_fwd, context_attention_fwd_mepic,
                        check_device, device_status, launch_count, reserve_workspace)

__all__ = [
    "reserve_workspace",
    "MAX_PACKED_Q_OFFSET", "LazyMetadataBuffers", "max_rotation_offset",
    "metadata_for_lazy_attention", "metadata_for_mepic", "metadata_for_variant",
    "pack_block_table", "validate_rotation_offsets", "ROPE_DEFAULT",
    "ROPE_LLAMA3", "build_cos_sin_table", "rope_meta_from_layer",
    "chunked_prefill_paged_decode", "chunked_prefill_paged_decode_mepic",
    "context_attention_fwd", "context_attention_fwd_mepic", "launch_count",
    "device_status", "check_device", "write_to_paged_cache",
]
