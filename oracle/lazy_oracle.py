"""CPU oracle for the deferred-RoPE attention path.  TEST INFRASTRUCTURE ONLY.

This module is a float32 torch / numpy restatement of the reference's
algorithm.  It exists to check the CUDA kernels; it is never the thing that is
shipped or measured as the product.  Only ``tests/``, ``__graft_entry__.smoke``
and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import
it.  Nothing under ``lazy_attention_b200/`` does.

Parity status: PINNED.  The integer functions are checked against the golden
vectors of the reference's own tests (lazy_attn/tests/core/test_scheduler.py:36-61,
tests/core/test_rotation_offset_bound.py:19-75, tests/worker/test_q_offset_range.py:54-79);
the floating-point functions are checked against fixtures produced by running
the reference's own Triton kernels under the Triton CPU interpreter
(tests/golden/make_golden.py wrote tests/golden/*.npz).

Each function cites the reference file:line it restates (paths relative to the
reference repository root).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch

MAX_PACKED_Q_OFFSET = 0xFFFF  # lazy_attn/lazy/utils/rotation.py:15

ROPE_DEFAULT = 0  # lazy_attn/lazy/model_executor/rope/cos_sin.py:20
ROPE_LLAMA3 = 1   # lazy_attn/lazy/model_executor/rope/cos_sin.py:21


# --------------------------------------------------------------------------
# Integer path (bit-exact)
# --------------------------------------------------------------------------
def metadata_for_lazy_attention(document_lens: Sequence[int],
                                document_lens_padded: Sequence[int],
                                block_size: int):
    """lazy_attn/lazy/core/sched/scheduler.py:758-781.

    One entry per document page plus one trailing entry for the query page.
    q_offset is the +1-biased rotation position (total padding plus the true
    lengths of all earlier documents); q_mask is the pad count, recorded on the
    last page of each document.  Returns two python lists of ints.
    """
    num_blocks = sum(document_lens_padded) // block_size + 1
    q_mask = np.zeros(num_blocks, dtype=np.int32)
    q_offset = np.zeros(num_blocks, dtype=np.int32)
    pads = np.array(document_lens_padded) - np.array(document_lens)
    pos = int(pads.sum()) if len(pads) else 0
    cursor = 0
    for d in range(len(document_lens)):
        n = document_lens_padded[d] // block_size
        q_offset[cursor:cursor + n] = pos + 1
        cursor += n
        q_mask[cursor - 1] = pads[d]
        pos += document_lens[d]
    q_offset[cursor] = 1
    return [int(v) for v in q_offset], [int(v) for v in q_mask]


def metadata_for_mepic(document_lens, document_lens_padded, block_size):
    """lazy_attn/lazy/core/sched/scheduler.py:784-787: offsets zeroed, same mask."""
    q_offset, q_mask = metadata_for_lazy_attention(document_lens,
                                                   document_lens_padded,
                                                   block_size)
    return [0 for _ in q_offset], q_mask


def max_rotation_offset(document_lens, document_lens_padded) -> int:
    """lazy_attn/lazy/utils/rotation.py:18-37."""
    if not document_lens:
        return 0
    pad = sum(p - t for t, p in zip(document_lens, document_lens_padded))
    return pad + sum(document_lens[:-1]) + 1


def pack_block_table(block_table: np.ndarray, q_offset: np.ndarray,
                     q_mask: np.ndarray) -> np.ndarray:
    """lazy_attn/lazy/worker/gpu_model_runner.py:322-330.

    packed = (block_id.int64 << 32) | (q_offset.int64 << 16) | q_mask.int64,
    with the same unchecked carry behaviour as the reference when a field is
    too wide (the reference refuses q_offset > 0xFFFF earlier, at :217-225).
    """
    bt = np.asarray(block_table).astype(np.int64)
    off = np.asarray(q_offset).astype(np.int64)
    msk = np.asarray(q_mask).astype(np.int64)
    return (bt << 32) | (off << 16) | msk


def unpack_block_table(packed: np.ndarray):
    """lazy_attn/lazy/attention/ops/models/llama_v1.py:157-160."""
    p = np.asarray(packed).astype(np.int64)
    blk = (p >> 32).astype(np.int32)
    rot = ((p >> 16) & 0xFFFF).astype(np.int32)
    pad = (p & 0xFFFF).astype(np.int32)
    return blk, rot, pad


# --------------------------------------------------------------------------
# cos/sin table
# --------------------------------------------------------------------------
def rope_inv_freq(rotary_dim: int, base: float, rope_type: int = ROPE_DEFAULT,
                  scaling_factor: float = 1.0, low_freq_factor: float = 1.0,
                  high_freq_factor: float = 1.0,
                  orig_max_position: int = 8192) -> torch.Tensor:
    """lazy_attn/lazy/model_executor/rope/cos_sin.py:24-59 and :127-145.

    float32 inverse frequencies, length rotary_dim // 2, optionally with the
    llama3 wavelength-dependent smoothing.
    """
    idx = torch.arange(0, rotary_dim, 2, dtype=torch.float32)
    inv = 1.0 / (base ** (idx / rotary_dim))
    if rope_type == ROPE_LLAMA3:
        wave_len = 2 * math.pi / inv
        low_wl = orig_max_position / low_freq_factor
        high_wl = orig_max_position / high_freq_factor
        if high_freq_factor != low_freq_factor:
            smooth = (orig_max_position / wave_len - low_freq_factor) / (
                high_freq_factor - low_freq_factor)
        else:
            smooth = torch.zeros_like(inv)
        inv = torch.where(
            wave_len < high_wl, inv,
            torch.where(wave_len > low_wl, inv / scaling_factor,
                        (1 - smooth) * inv / scaling_factor + smooth * inv))
    return inv


def build_cos_sin_table(max_position: int, rotary_dim: int, base: float,
                        rope_type: int = ROPE_DEFAULT,
                        scaling_factor: float = 1.0,
                        low_freq_factor: float = 1.0,
                        high_freq_factor: float = 1.0,
                        orig_max_position: int = 8192) -> torch.Tensor:
    """Row ``pos`` = [cos(pos*inv) (rotary_dim/2) | sin(pos*inv) (rotary_dim/2)].

    Layout consumed by every kernel of the path
    (lazy_attn/lazy/attention/ops/models/llama_v1.py:216-221,
    lazy_attn/lazy/attention/ops/prefix_prefill.py:186-190); values follow
    lazy_attn/lazy/model_executor/rope/cos_sin.py:62-66.  float32.
    """
    inv = rope_inv_freq(rotary_dim, base, rope_type, scaling_factor,
                        low_freq_factor, high_freq_factor, orig_max_position)
    t = torch.arange(max_position, dtype=torch.float32)
    theta = t[:, None] * inv[None, :]
    return torch.cat([torch.cos(theta), torch.sin(theta)], dim=-1)


# --------------------------------------------------------------------------
# Paged cache helpers
# --------------------------------------------------------------------------
def _fp8_dtype(kv_cache_dtype: str):
    if kv_cache_dtype in ("fp8", "fp8_e4m3"):
        return torch.float8_e4m3fn
    if kv_cache_dtype == "fp8_e5m2":
        return torch.float8_e5m2
    raise ValueError("Unsupported FP8 dtype:", kv_cache_dtype)


def _view_caches(kv_cache_dtype, k_cache, v_cache):
    """lazy_attn/lazy/attention/ops/prefix_prefill.py:637-654."""
    if "fp8" in kv_cache_dtype:
        assert k_cache.dtype == torch.uint8 and v_cache.dtype == torch.uint8
        dt = _fp8_dtype(kv_cache_dtype)
        k_cache = k_cache.view(dt)
        v_cache = v_cache.view(dt)
    if k_cache.dtype == torch.uint8 or (v_cache.dtype == torch.uint8
                                        and kv_cache_dtype == "auto"):
        raise ValueError("kv_cache_dtype='auto' unsupported for FP8 KV Cache")
    return k_cache, v_cache


def gather_pages(k_cache, v_cache, block_ids, k_scale=1.0, v_scale=1.0):
    """Un-page K and V for a list of physical blocks.

    K cache is [nb, Hkv, D/x, BS, x], V cache is [nb, Hkv, D, BS]
    (lazy_attn/lazy/attention/ops/models/llama_v1.py:22-23).  Returns float32
    K [Hkv, n*BS, D] and V [Hkv, n*BS, D]; fp8 caches are dequantised as
    ``float(x) * scale`` (lazy_attn/lazy/attention/ops/prefix_prefill.py:238-243).
    """
    idx = torch.as_tensor(block_ids, dtype=torch.long)
    if k_cache.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        k_scale = v_scale = 1.0  # the scales only apply to fp8 caches
    kb = k_cache[idx].to(torch.float32)  # [n, Hkv, D/x, BS, x]
    vb = v_cache[idx].to(torch.float32)  # [n, Hkv, D, BS]
    n, hkv, dx, bs, x = kb.shape
    k = kb.permute(1, 0, 3, 2, 4).reshape(hkv, n * bs, dx * x) * float(k_scale)
    v = vb.permute(1, 0, 3, 2).reshape(hkv, n * bs, dx * x) * float(v_scale)
    return k, v


def _rot_fwd(k, cos, sin):
    """K forward rotation, NeoX halves
    (lazy_attn/lazy/attention/ops/prefix_prefill.py:252-256)."""
    h = k.shape[-1] // 2
    k1, k2 = k[..., :h], k[..., h:]
    return torch.cat([k1 * cos - k2 * sin, k1 * sin + k2 * cos], dim=-1)


def _softmax_av(scores, v):
    """scores [H, M, N] (may contain -inf), v [H, N, D] -> [H, M, D]."""
    p = torch.softmax(scores, dim=-1)
    return torch.matmul(p, v)


# --------------------------------------------------------------------------
# Prefix-prefill, lazy variant
# --------------------------------------------------------------------------
def context_attention_fwd(q, k, v, o, kv_cache_dtype, k_cache, v_cache, b_loc,
                          b_start_loc, b_seq_len, max_seq_len, max_input_len,
                          k_scale, v_scale, alibi_slopes=None,
                          sliding_window=None, sm_scale=None,
                          skip_decode=False, cos_sin_cache=None,
                          rotary_dim=None, is_neox_style=True, is_lazy=None,
                          q_offset=None, q_mask=None):
    """Restates lazy_attn/lazy/attention/ops/prefix_prefill.py:34-744.

    Per request: cached context pages are read through ``b_loc``; for a lazy
    request each page's K is rotated forward by ``q_offset-1`` (0 and 1 both
    mean identity, :180-190) and the last ``q_mask`` tokens of the page are
    masked (:267-271); a non-lazy request uses the plain branch (:398-592).
    The new tokens attend causally to the un-rotated new K/V (:325-385).
    Writes ``o`` in place (float32 math, cast to ``o.dtype`` at the end).
    """
    if alibi_slopes is not None:
        raise NotImplementedError(
            "Alibi slopes are not implemented for prefix prefill")
    k_cache, v_cache = _view_caches(kv_cache_dtype, k_cache, v_cache)
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    BS = v_cache.shape[3]
    if sm_scale is None:
        sm_scale = 1.0 / (D ** 0.5)
    sw = 0 if sliding_window is None or sliding_window <= 0 else int(sliding_window)
    ks, vs = float(k_scale), float(v_scale)
    cs = None if cos_sin_cache is None else cos_sin_cache.to(torch.float32)
    half = D // 2
    B = b_seq_len.shape[0]
    assert B + 1 == len(b_start_loc)
    for b in range(B):
        s0, s1 = int(b_start_loc[b]), int(b_start_loc[b + 1])
        qlen = s1 - s0
        ctx = int(b_seq_len[b]) - qlen
        if qlen <= 0 or (skip_decode and qlen == 1):
            continue
        lazy = bool(is_lazy[b]) if is_lazy is not None else False
        npages = (ctx + BS - 1) // BS
        qf = q[s0:s1].to(torch.float32).permute(1, 0, 2)  # [Hq, M, D]
        score_parts, v_parts = [], []
        if npages:
            blocks = [int(b_loc[b, j]) for j in range(npages)]
            kc, vc = gather_pages(k_cache, v_cache, blocks, ks, vs)
            tok = torch.arange(npages * BS)
            page = tok // BS
            valid = tok < ctx
            if lazy:
                rot = torch.as_tensor([int(q_offset[b, j]) for j in range(npages)])
                pos = torch.where(rot != 0, rot - 1, torch.zeros_like(rot))
                cos = cs[pos][:, :half][page]   # [N, D/2]
                sin = cs[pos][:, half:][page]
                kc = _rot_fwd(kc, cos[None], sin[None])
                pad = torch.as_tensor([int(q_mask[b, j]) for j in range(npages)])
                bound = torch.minimum(torch.tensor(ctx), (page + 1) * BS - pad[page])
                valid = tok < bound
            kc = kc.repeat_interleave(G, dim=0)
            sc = torch.matmul(qf, kc.transpose(1, 2))
            sc = torch.where(valid[None, None, :], sc, torch.tensor(float("-inf")))
            sc = sc * sm_scale
            if sw > 0:
                qpos = ctx + torch.arange(qlen)
                far = (qpos[:, None] - tok[None, :]) >= sw
                sc = torch.where(far[None], torch.tensor(-10000.0), sc)
            score_parts.append(sc)
            v_parts.append(vc.repeat_interleave(G, dim=0))
        kn = k[s0:s1].to(torch.float32).permute(1, 0, 2).repeat_interleave(G, dim=0)
        vn = v[s0:s1].to(torch.float32).permute(1, 0, 2).repeat_interleave(G, dim=0)
        sc = torch.matmul(qf, kn.transpose(1, 2)) * sm_scale
        m_idx = torch.arange(qlen)
        causal = m_idx[:, None] >= m_idx[None, :]
        sc = torch.where(causal[None], sc, torch.tensor(float("-inf")))
        if sw > 0:
            far = (m_idx[:, None] - m_idx[None, :]) >= sw
            sc = torch.where(far[None], torch.tensor(-10000.0), sc)
        score_parts.append(sc)
        v_parts.append(vn)
        out = _softmax_av(torch.cat(score_parts, dim=-1), torch.cat(v_parts, dim=1))
        o[s0:s1] = out.permute(1, 0, 2).to(o.dtype)


# --------------------------------------------------------------------------
# Prefix-prefill, per-token ("mepic") variant
# --------------------------------------------------------------------------
def context_attention_fwd_mepic(q, k, v, o, kv_cache_dtype, k_cache, v_cache,
                                b_loc, b_start_loc, b_seq_len, max_seq_len,
                                max_input_len, k_scale, v_scale,
                                alibi_slopes=None, sliding_window=None,
                                sm_scale=None, skip_decode=False,
                                cos_sin_cache=None, rotary_dim=None,
                                is_neox_style=True, q_mask=None, q_offset=None,
                                is_mepic: bool = True,
                                force_fp32_rotary: bool = False):
    """Restates lazy_attn/lazy/attention/old_ops/prefix_prefill.py:34-555.

    Cached K is un-rotated; every cached token is rotated at its own position:
    the absolute slot ``j*BS+t`` when ``is_mepic`` (:183-184), otherwise
    ``(q_offset-1 or page start) + t`` (:186-191).  The new K is rotated at
    ``ctx_len + n`` (:342-365).  Padding is masked by q_mask (:165-167,262).
    """
    if alibi_slopes is not None:
        raise NotImplementedError(
            "Alibi slopes are not implemented for prefix prefill")
    k_cache, v_cache = _view_caches(kv_cache_dtype, k_cache, v_cache)
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    BS = v_cache.shape[3]
    if sm_scale is None:
        sm_scale = 1.0 / (D ** 0.5)
    sw = 0 if sliding_window is None or sliding_window <= 0 else int(sliding_window)
    ks, vs = float(k_scale), float(v_scale)
    cs = cos_sin_cache.to(torch.float32)
    half = D // 2
    B = b_seq_len.shape[0]
    for b in range(B):
        s0, s1 = int(b_start_loc[b]), int(b_start_loc[b + 1])
        qlen = s1 - s0
        ctx = int(b_seq_len[b]) - qlen
        if qlen <= 0 or (skip_decode and qlen == 1):
            continue
        npages = (ctx + BS - 1) // BS
        qf = q[s0:s1].to(torch.float32).permute(1, 0, 2)
        score_parts, v_parts = [], []
        if npages:
            blocks = [int(b_loc[b, j]) for j in range(npages)]
            kc, vc = gather_pages(k_cache, v_cache, blocks, ks, vs)
            tok = torch.arange(npages * BS)
            page = tok // BS
            lane = tok % BS
            if is_mepic:
                pos = tok
            else:
                rot = torch.as_tensor([int(q_offset[b, j]) for j in range(npages)])
                base = torch.where(rot != 0, rot - 1, torch.arange(npages) * BS)
                pos = base[page] + lane
            pad = torch.as_tensor([int(q_mask[b, j]) for j in range(npages)])
            bound = torch.minimum(torch.tensor(ctx), (page + 1) * BS - pad[page])
            valid = tok < bound
            pos = torch.where(valid, pos, torch.zeros_like(pos))
            cos = cs[pos][:, :half]
            sin = cs[pos][:, half:]
            kc = _rot_fwd(kc, cos[None], sin[None]).repeat_interleave(G, dim=0)
            sc = torch.matmul(qf, kc.transpose(1, 2))
            sc = torch.where(valid[None, None, :], sc, torch.tensor(float("-inf")))
            sc = sc * sm_scale
            if sw > 0:
                qpos = ctx + torch.arange(qlen)
                far = (qpos[:, None] - tok[None, :]) >= sw
                sc = torch.where(far[None], torch.tensor(-10000.0), sc)
            score_parts.append(sc)
            v_parts.append(vc.repeat_interleave(G, dim=0))
        kn = k[s0:s1].to(torch.float32).permute(1, 0, 2)
        npos = ctx + torch.arange(qlen)
        kn = _rot_fwd(kn, cs[npos][None, :, :half], cs[npos][None, :, half:])
        kn = kn.repeat_interleave(G, dim=0)
        vn = v[s0:s1].to(torch.float32).permute(1, 0, 2).repeat_interleave(G, dim=0)
        sc = torch.matmul(qf, kn.transpose(1, 2)) * sm_scale
        m_idx = torch.arange(qlen)
        causal = m_idx[:, None] >= m_idx[None, :]
        sc = torch.where(causal[None], sc, torch.tensor(float("-inf")))
        if sw > 0:
            far = (m_idx[:, None] - m_idx[None, :]) >= sw
            sc = torch.where(far[None], torch.tensor(-10000.0), sc)
        score_parts.append(sc)
        v_parts.append(vn)
        out = _softmax_av(torch.cat(score_parts, dim=-1), torch.cat(v_parts, dim=1))
        o[s0:s1] = out.permute(1, 0, 2).to(o.dtype)


# --------------------------------------------------------------------------
# Decode, lazy variant (query-side rotation, packed table)
# --------------------------------------------------------------------------
def paged_decode_lazy(output, query, key_cache, value_cache, packed_block_table,
                      seq_lens, query_start_loc, sm_scale, k_scale, v_scale,
                      cos_sin_cache, is_lazy, kv_cache_dtype="auto",
                      alibi_slopes=None, sliding_window=0,
                      ignore_q_mask=False, round_q_to=None):
    """Restates lazy_attn/lazy/attention/ops/models/llama_v1.py:85-434.

    One query token per sequence; sequences whose query length exceeds 1 are
    left untouched (:93-100).  Per page the packed entry gives the physical
    block, the +1-biased rotation offset and the pad count (:157-160).  When
    the offset differs from the previous page's: 1 restores the original Q, a
    value >1 rebuilds Q from the original by the inverse rotation at
    ``offset-1``, 0 keeps the current Q (:206-238).  ``round_q_to`` optionally
    rounds the rotated Q to a storage dtype as the reference does (:235-237).
    Non-lazy sequences still read the block id from the high half (:345-346).
    """
    key_cache, value_cache = _view_caches(kv_cache_dtype, key_cache, value_cache)
    Hq, D = query.shape[1], query.shape[2]
    Hkv = key_cache.shape[1]
    G = Hq // Hkv
    BS = value_cache.shape[3]
    half = D // 2
    ks, vs = float(k_scale), float(v_scale)
    cs = None if cos_sin_cache is None else cos_sin_cache.to(torch.float32)
    sw = 0 if sliding_window is None or sliding_window <= 0 else int(sliding_window)
    blk_all, rot_all, pad_all = unpack_block_table(
        packed_block_table.cpu().numpy() if torch.is_tensor(packed_block_table)
        else packed_block_table)
    num_seqs = len(seq_lens)
    for s in range(num_seqs):
        s0, s1 = int(query_start_loc[s]), int(query_start_loc[s + 1])
        if s1 - s0 != 1:
            continue
        L = int(seq_lens[s])
        npages = (L + BS - 1) // BS
        if npages == 0:
            continue
        lazy = bool(is_lazy[s]) if is_lazy is not None else False
        blocks = [int(blk_all[s, j]) for j in range(npages)]
        kc, vc = gather_pages(key_cache, value_cache, blocks, ks, vs)
        q0 = query[s0].to(torch.float32)  # [Hq, D]
        tok = torch.arange(npages * BS)
        page = tok // BS
        lane = tok % BS
        valid = tok < L
        if lazy:
            if not ignore_q_mask:
                pad = torch.as_tensor(pad_all[s, :npages].astype(np.int64))
                valid = valid & (lane < (BS - pad[page]))
            # per-page rotated query
            q_pages = torch.empty(npages, Hq, D)
            cur = q0
            prev = -1
            for j in range(npages):
                r = int(rot_all[s, j])
                if r != prev:
                    if r == 1:
                        cur = q0
                    elif r != 0:
                        c, sn = cs[r - 1, :half], cs[r - 1, half:]
                        q1, q2 = q0[:, :half], q0[:, half:]
                        cur = torch.cat([q1 * c + q2 * sn, -q1 * sn + q2 * c], dim=-1)
                        if round_q_to is not None:
                            cur = cur.to(round_q_to).to(torch.float32)
                    prev = r
                q_pages[j] = cur
            qtok = q_pages[page]  # [N, Hq, D]
            kq = kc.repeat_interleave(G, dim=0).permute(1, 0, 2)  # [N, Hq, D]
            sc = (qtok * kq).sum(-1).t()  # [Hq, N]
        else:
            sc = torch.einsum("hd,hnd->hn", q0, kc.repeat_interleave(G, dim=0))
        sc = sc * sm_scale
        sc = torch.where(valid[None], sc, torch.tensor(float("-inf")))
        ctx_len = L - 1
        if sw > 0:
            sc = torch.where(((ctx_len - tok) < sw)[None], sc, torch.tensor(-10000.0))
        if alibi_slopes is not None:
            sc = sc + alibi_slopes.to(torch.float32)[:, None] * (tok - ctx_len)[None].float()
        p = torch.softmax(sc, dim=-1)
        out = torch.einsum("hn,hnd->hd", p, vc.repeat_interleave(G, dim=0))
        output[s0] = out.to(output.dtype)


# --------------------------------------------------------------------------
# Decode, per-token ("mepic") variant
# --------------------------------------------------------------------------
def paged_decode_mepic(output, query, key_cache, value_cache, block_table,
                       q_mask, seq_lens, query_start_loc, sm_scale, k_scale,
                       v_scale, cos_sin_cache, kv_cache_dtype="auto",
                       alibi_slopes=None, sliding_window=0):
    """Restates lazy_attn/lazy/attention/old_ops/chunked_prefill_paged_decode.py:69-280.

    Plain int32 block table and q_mask (:140-141); every cached token's K is
    rotated at its slot position ``j*BS+t`` (:204-233); masks as the lazy
    decode (:197-201).
    """
    key_cache, value_cache = _view_caches(kv_cache_dtype, key_cache, value_cache)
    Hq, D = query.shape[1], query.shape[2]
    Hkv = key_cache.shape[1]
    G = Hq // Hkv
    BS = value_cache.shape[3]
    half = D // 2
    ks, vs = float(k_scale), float(v_scale)
    cs = cos_sin_cache.to(torch.float32)
    sw = 0 if sliding_window is None or sliding_window <= 0 else int(sliding_window)
    for s in range(len(seq_lens)):
        s0, s1 = int(query_start_loc[s]), int(query_start_loc[s + 1])
        if s1 - s0 != 1:
            continue
        L = int(seq_lens[s])
        npages = (L + BS - 1) // BS
        if npages == 0:
            continue
        blocks = [int(block_table[s, j]) for j in range(npages)]
        kc, vc = gather_pages(key_cache, value_cache, blocks, ks, vs)
        tok = torch.arange(npages * BS)
        page = tok // BS
        lane = tok % BS
        pad = torch.as_tensor([int(q_mask[s, j]) for j in range(npages)])
        valid = (tok < L) & (lane < (BS - pad[page]))
        kc = _rot_fwd(kc, cs[tok][None, :, :half], cs[tok][None, :, half:])
        q0 = query[s0].to(torch.float32)
        sc = torch.einsum("hd,hnd->hn", q0, kc.repeat_interleave(G, dim=0)) * sm_scale
        sc = torch.where(valid[None], sc, torch.tensor(float("-inf")))
        ctx_len = L - 1
        if sw > 0:
            sc = torch.where(((ctx_len - tok) < sw)[None], sc, torch.tensor(-10000.0))
        if alibi_slopes is not None:
            sc = sc + alibi_slopes.to(torch.float32)[:, None] * (tok - ctx_len)[None].float()
        p = torch.softmax(sc, dim=-1)
        out = torch.einsum("hn,hnd->hd", p, vc.repeat_interleave(G, dim=0))
        output[s0] = out.to(output.dtype)


# --------------------------------------------------------------------------
# Dispatch wrappers (same argument surface as the reference)
# --------------------------------------------------------------------------
def chunked_prefill_paged_decode(query, key, value, output, kv_cache_dtype,
                                 key_cache, value_cache, block_table,
                                 query_start_loc, seq_lens, max_seq_len,
                                 max_query_len, k_scale, v_scale,
                                 alibi_slopes=None, sliding_window=None,
                                 sm_scale=None, rotary_dim=None, freqs=None,
                                 cos_sin_cache=None, rope_meta=None,
                                 is_neox_style=True, is_lazy=None,
                                 lazy_variant=None, q_offset=None, q_mask=None,
                                 packed_block_table=None, round_q_to=None):
    """Restates lazy_attn/lazy/attention/ops/chunked_prefill_paged_decode.py:36-221.

    Keeps the reference's default scale quirk: ``1/sqrt(query.shape[1])`` (the
    number of heads, :71-72).  Prefill runs when ``max_query_len > 1`` (:79-106),
    the decode kernel always runs and skips sequences with more than one query
    token.  The decode table is the packed one when given (:165-167).
    """
    if sm_scale is None:
        sm_scale = 1.0 / (query.shape[1] ** 0.5)
    if max_query_len > 1:
        context_attention_fwd(query, key, value, output, kv_cache_dtype,
                              key_cache, value_cache, block_table,
                              query_start_loc, seq_lens, max_seq_len,
                              max_query_len, k_scale, v_scale,
                              alibi_slopes=alibi_slopes,
                              sliding_window=sliding_window, sm_scale=sm_scale,
                              skip_decode=True, cos_sin_cache=cos_sin_cache,
                              rotary_dim=rotary_dim, is_neox_style=is_neox_style,
                              is_lazy=is_lazy, q_offset=q_offset, q_mask=q_mask)
    table = packed_block_table if packed_block_table is not None else block_table
    paged_decode_lazy(output, query, key_cache, value_cache, table, seq_lens,
                      query_start_loc, sm_scale, k_scale, v_scale,
                      cos_sin_cache, is_lazy, kv_cache_dtype=kv_cache_dtype,
                      alibi_slopes=alibi_slopes, sliding_window=sliding_window,
                      round_q_to=round_q_to)


def chunked_prefill_paged_decode_mepic(query, key, value, output, kv_cache_dtype,
                                       key_cache, value_cache, block_table,
                                       query_start_loc, seq_lens, max_seq_len,
                                       max_query_len, k_scale, v_scale,
                                       alibi_slopes=None, sliding_window=None,
                                       sm_scale=None, rotary_dim=None,
                                       cos_sin_cache=None, is_neox_style=True,
                                       q_offset=None, q_mask=None,
                                       is_mepic: bool = True,
                                       force_fp32_rotary: bool = False):
    """Restates lazy_attn/lazy/attention/old_ops/chunked_prefill_paged_decode.py:283-442."""
    if sm_scale is None:
        sm_scale = 1.0 / (query.shape[1] ** 0.5)
    if q_mask is None:
        q_mask = torch.zeros_like(block_table, dtype=torch.int32)
    if q_offset is None:
        q_offset = torch.zeros_like(block_table, dtype=torch.int32)
    if max_query_len > 1:
        context_attention_fwd_mepic(query, key, value, output, kv_cache_dtype,
                                    key_cache, value_cache, block_table,
                                    query_start_loc, seq_lens, max_seq_len,
                                    max_query_len, k_scale, v_scale,
                                    alibi_slopes=alibi_slopes,
                                    sliding_window=sliding_window,
                                    sm_scale=sm_scale, skip_decode=True,
                                    cos_sin_cache=cos_sin_cache,
                                    rotary_dim=rotary_dim,
                                    is_neox_style=is_neox_style, q_mask=q_mask,
                                    q_offset=q_offset, is_mepic=is_mepic,
                                    force_fp32_rotary=force_fp32_rotary)
    paged_decode_mepic(output, query, key_cache, value_cache, block_table,
                       q_mask, seq_lens, query_start_loc, sm_scale, k_scale,
                       v_scale, cos_sin_cache, kv_cache_dtype=kv_cache_dtype,
                       alibi_slopes=alibi_slopes, sliding_window=sliding_window)


# --------------------------------------------------------------------------
# Paged-cache write (the step before the attention op)
# --------------------------------------------------------------------------
def write_to_paged_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype,
                         k_scale, v_scale):
    """Restates what the reference's backend asks of vLLM 0.9.2 before the op
    (lazy_attn/lazy/attention/backends/triton_attn.py:100-109): token ``t`` goes to
    page ``slot // BS``, in-page index ``slot % BS``, in the cache layouts the
    reference documents (lazy_attn/lazy/attention/ops/models/llama_v1.py:22-23);
    an fp8 cache stores ``fp8(x / scale)`` (saturating).  Parity unpinned: the
    callee is third-party (vLLM ``reshape_and_cache``) and no reference test holds
    vectors for it.  Modifies the caches in place.
    """
    kc, vc = _view_caches(kv_cache_dtype, key_cache, value_cache)
    nb, hkv, dx, bs, x = kc.shape
    fp8 = kc.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
    ks = float(k_scale) if fp8 else 1.0
    vs = float(v_scale) if fp8 else 1.0
    for t in range(min(key.shape[0], slot_mapping.shape[0])):
        slot = int(slot_mapping[t])
        if slot < 0:
            continue
        blk, off = slot // bs, slot % bs
        kt = key[t].to(torch.float32) / ks if fp8 else key[t]
        vt = value[t].to(torch.float32) / vs if fp8 else value[t]
        if fp8:
            lim = torch.finfo(kc.dtype).max
            kt, vt = kt.clamp(-lim, lim), vt.clamp(-lim, lim)
        kc[blk, :, :, off, :] = kt.reshape(hkv, dx, x).to(kc.dtype)
        vc[blk, :, :, off] = vt.to(vc.dtype)


# --------------------------------------------------------------------------
# The query-only rotary op that precedes the attention op
# --------------------------------------------------------------------------
def apply_rotary_q(query, positions, cos_sin_cache):
    """lazy_attn/lazy/model_executor/layers/rotary_embedding.py:40-66 (query path).

    NeoX style on the full head: ``cos, sin = cos_sin_cache[positions].chunk(2)``;
    ``o1 = x1*cos - x2*sin``, ``o2 = x2*cos + x1*sin`` over the two halves of each
    head.  float32 math on float32 copies of the inputs; the result is rounded to
    ``query.dtype`` (the op writes the query tensor in place).  The key is not
    rotated: the attention kernels rotate the cached keys themselves.
    """
    q = query.to(torch.float32)
    cs = cos_sin_cache.to(torch.float32)[positions.to(torch.long)]   # [T, rd]
    half = cs.shape[-1] // 2
    cos, sin = cs[:, None, :half], cs[:, None, half:]
    x1, x2 = q[..., :half], q[..., half:2 * half]
    out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, q[..., 2 * half:]], dim=-1)
    return out.to(query.dtype)
