"""CPU restatement of the Native Sparse Attention operators (TEST INFRASTRUCTURE ONLY).

This module is the checker for the CUDA kernels of this repository.  It is never
imported by the product package: only the tests, the smoke entry and the CPU
baseline leg of the benchmark may use it.

Every function restates, in plain fp32 torch (on the CPU; the tensors' device is
followed, so a test may also evaluate it on a GPU in true fp32) what the reference project
(XunhaoLai/native-sparse-attention-triton) computes.  The reference file and
lines each function follows are cited in its docstring (paths are relative to
the reference project root).  The restatement is pinned against the reference's
own ``ops.torch`` implementations by the fixtures in ``tests/golden`` made by
``tests/golden/make_golden.py`` (which imports the reference on the CPU), and
against the reference ITSELF run on a B200 -- its Triton operators, the
flash_attn call of its sliding-window branch, its RotaryEmbedding, its nsa_infer
with its NSACache -- by the ``box_*.npz`` fixtures made by
``tests/golden/make_golden_on_box.py``.

All functions are differentiable torch code, so gradients for the backward
parity tests come from autograd over these fp32 formulas.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch


# --------------------------------------------------------------------------- #
# sequence-length helpers
# --------------------------------------------------------------------------- #
def compressed_seqlens(cu_seqlens: torch.Tensor, kernel_size: int, kernel_stride: int):
    """``(y_seqlens, y_cu_seqlens)`` after strided-window compression.

    Follows native_sparse_attention/ops/triton/utils.py:25-37: a sequence of
    length L gives ``(L - kernel_size) // kernel_stride + 1`` windows, and none
    at all when ``L < kernel_size``.
    """
    seqlens = (cu_seqlens[1:] - cu_seqlens[:-1]).to(torch.int64)
    y = torch.div(seqlens - kernel_size, kernel_stride, rounding_mode="floor") + 1
    y = torch.where(seqlens < kernel_size, torch.zeros_like(y), y)
    y_cu = torch.zeros(y.numel() + 1, dtype=torch.int32, device=cu_seqlens.device)
    y_cu[1:] = torch.cumsum(y, 0).to(torch.int32)
    return y.to(torch.int32), y_cu


def _windows(x_seq: torch.Tensor, n_win: int, kernel_size: int, kernel_stride: int):
    """[L, H, d] -> [n_win, kernel_size, H, d] view of the strided windows."""
    L, H, d = x_seq.shape
    return x_seq.as_strided(
        (n_win, kernel_size, H, d),
        (kernel_stride * x_seq.stride(0), x_seq.stride(0), x_seq.stride(1), x_seq.stride(2)),
    )


# --------------------------------------------------------------------------- #
# compression (rows a1 / a2 of the hot-path table)
# --------------------------------------------------------------------------- #
def linear_compress(x, w, cu_seqlens, kernel_size, kernel_stride, pe=None):
    """``y[m,h,:] = concat_k(x[s+m*stride+k,h,:]) @ w[h]`` plus ``concat_k(pe[h,k,:]) @ w[h]``.

    Follows native_sparse_attention/ops/torch/compress_key_value.py:190-231
    (window view -> einsum with ``w`` reshaped ``h (k d) D`` -> bias from ``pe``).
    """
    N, H, d = x.shape
    y_len, y_cu = compressed_seqlens(cu_seqlens, kernel_size, kernel_stride)
    wk = w.reshape(H, kernel_size, d, -1)
    outs = []
    for b in range(y_len.numel()):
        s, m = int(cu_seqlens[b]), int(y_len[b])
        if m == 0:
            continue
        win = _windows(x[s : int(cu_seqlens[b + 1])], m, kernel_size, kernel_stride)
        outs.append(torch.einsum("nkhd,hkdD->nhD", win, wk))
    y = torch.cat(outs, 0) if outs else x.new_zeros(0, H, w.shape[-1])
    if pe is not None:
        bias = torch.einsum("hD,hDd->hd", pe.reshape(H, -1), w)
        y = y + bias.unsqueeze(0)
    return y, y_cu


def weightedpool_compress(x, w, cu_seqlens, kernel_size, kernel_stride, pe=None):
    """``y[m,h,:] = sum_k w[h,k] * x[s+m*stride+k,h,:]`` plus ``sum_k w[h,k]*pe[h,k,:]``.

    Follows native_sparse_attention/ops/torch/compress_key_value.py:117-153.
    """
    N, H, d = x.shape
    y_len, y_cu = compressed_seqlens(cu_seqlens, kernel_size, kernel_stride)
    outs = []
    for b in range(y_len.numel()):
        s, m = int(cu_seqlens[b]), int(y_len[b])
        if m == 0:
            continue
        win = _windows(x[s : int(cu_seqlens[b + 1])], m, kernel_size, kernel_stride)
        outs.append(torch.einsum("nkhd,hk->nhd", win, w))
    y = torch.cat(outs, 0) if outs else x.new_zeros(0, H, d)
    if pe is not None:
        y = y + torch.einsum("hkd,hk->hd", pe, w).unsqueeze(0)
    return y, y_cu


def avgpool_compress(x, w, cu_seqlens, kernel_size, kernel_stride, pe=None):
    """Mean over each window plus ``mean_k pe[h,k,:]``.

    Follows native_sparse_attention/ops/torch/compress_key_value.py:52-81.
    """
    assert w is None, "don't need additional weight for avgpool"
    H = x.shape[1]
    ww = x.new_full((H, kernel_size), 1.0 / kernel_size)
    y, y_cu = weightedpool_compress(x, ww, cu_seqlens, kernel_size, kernel_stride, None)
    if pe is not None:
        y = y + pe.mean(1).unsqueeze(0)
    return y, y_cu


# --------------------------------------------------------------------------- #
# block scores and top-k selection
# --------------------------------------------------------------------------- #
def block_score_weights(kernel_size: int, kernel_stride: int, block_size: int) -> List[int]:
    """Weights that turn compressed-key scores into selection-block scores.

    ``w[o] = #{(i, j): i < kernel_size/stride, j < block_size/stride, i + j = o}``;
    block ``b`` reads compressed key ``b*(block_size/stride) - (kernel_size/stride - 1) + o``.
    Follows native_sparse_attention/ops/triton/compressed_attention.py:1130-1143
    and ops/torch/compressed_attention.py:34-53.
    """
    a, c = kernel_size // kernel_stride, block_size // kernel_stride
    w = [0] * (a + c - 1)
    for i in range(a):
        for j in range(c):
            w[i + j] += 1
    return w


def block_scores_from_key_scores(score, kernel_size, kernel_stride, block_size, num_blocks):
    """score [..., Lk] (already summed over the query heads of a KV group) -> [..., num_blocks]."""
    a, c = kernel_size // kernel_stride, block_size // kernel_stride
    w = block_score_weights(kernel_size, kernel_stride, block_size)
    Lk = score.shape[-1]
    need = (num_blocks - 1) * c + len(w)  # index after left-padding by a-1
    padded = torch.nn.functional.pad(score, (a - 1, max(0, need - (a - 1) - Lk)))
    out = score.new_zeros(*score.shape[:-1], num_blocks)
    for o, wo in enumerate(w):
        out = out + wo * padded[..., o :: c][..., :num_blocks]
    return out


def select_topk_blocks(block_score, q_block, topk, init_blocks, local_blocks):
    """Top-k selection with forced blocks, ascending order, ``-1`` padding.

    block_score [..., Q, num_blocks] fp32; q_block [Q] = block id of each query.
    Blocks ``< init_blocks`` and blocks in ``(q_block - local_blocks, q_block]``
    score ``+inf``; ``topk = min(topk, num_blocks)``; picked ids are sorted and
    ids beyond the query's own block become ``-1``.  Follows
    native_sparse_attention/ops/triton/compressed_attention.py:1092-1100,1289-1292.
    """
    nb = block_score.shape[-1]
    b_idx = torch.arange(nb, device=block_score.device)
    forced = (b_idx[None, :] < init_blocks) | (
        (q_block[:, None] >= b_idx[None, :]) & (q_block[:, None] < b_idx[None, :] + local_blocks)
    )
    s = torch.where(forced, torch.full_like(block_score, float("inf")), block_score)
    k = min(topk, nb)
    idx = s.topk(k, dim=-1).indices.sort(-1).values
    idx = torch.where(idx > q_block[:, None], torch.full_like(idx, -1), idx)
    return idx.to(torch.int32), s


# --------------------------------------------------------------------------- #
# masked attention core: one KV head and one chunk of query rows at a time
# --------------------------------------------------------------------------- #
QUERY_CHUNK = 1024  # rows of logits held at once: [G, QUERY_CHUNK, Lk] fp32 per step


def _chunk_attention(qc, kh, vh, mask, sm_scale):
    """qc [c, G, d], kh/vh [Lk, d], mask bool [c, Lk] -> (out [c, G, d], p [G, c, Lk]); rows with no key give 0."""
    logits = torch.einsum("qgd,kd->gqk", qc, kh) * sm_scale
    logits = logits.masked_fill(~mask[None], float("-inf"))
    p = logits.softmax(-1).nan_to_num(0)
    return torch.einsum("gqk,kd->qgd", p, vh), p


def _masked_attention(q_seq, k_seq, v_seq, mask_fn, sm_scale, score_fn=None):
    """Softmax attention of one sequence with an arbitrary mask, evaluated per KV head and per chunk of QUERY_CHUNK
    query rows so that the memory in use is linear in the key length per chunk; chunks are re-evaluated in the
    backward pass (torch.utils.checkpoint) instead of being kept, so gradients cost no more memory than outputs.

    q_seq [Lq, Hq, d], k_seq/v_seq [Lk, Hkv, d] (any float dtype, any device); mask_fn(h, t0, t1) -> bool [t1-t0, Lk] for
    KV head h; score_fn(h, t0, t1, p_sum [t1-t0, Lk]) receives the probabilities summed over the head's query group.
    Returns fp32 [Lq, Hq, d]."""
    from torch.utils.checkpoint import checkpoint

    Lq, Hq, d = q_seq.shape
    Hkv = k_seq.shape[1]
    G = Hq // Hkv
    qf, kf, vf = q_seq.float(), k_seq.float(), v_seq.float()
    need_grad = torch.is_grad_enabled() and (qf.requires_grad or kf.requires_grad or vf.requires_grad)
    heads = []
    for h in range(Hkv):
        rows = []
        for t0 in range(0, Lq, QUERY_CHUNK):
            t1 = min(Lq, t0 + QUERY_CHUNK)
            qc, kh, vh = qf[t0:t1, h * G:(h + 1) * G], kf[:, h], vf[:, h]
            mask = mask_fn(h, t0, t1)
            if score_fn is not None:
                with torch.no_grad():
                    score_fn(h, t0, t1, _chunk_attention(qc, kh, vh, mask, sm_scale)[1].sum(0))
            if need_grad:
                out = checkpoint(lambda a, b, c, m=mask: _chunk_attention(a, b, c, m, sm_scale)[0], qc, kh, vh,
                                 use_reentrant=False)
            else:
                out = _chunk_attention(qc, kh, vh, mask, sm_scale)[0]
            rows.append(out)
        heads.append(torch.cat(rows, 0) if rows else qf.new_zeros(0, G, d))
    return torch.cat(heads, 1) if heads else qf.new_zeros(Lq, Hq, d)


# --------------------------------------------------------------------------- #
# attention between queries and compressed keys (row a3)
# --------------------------------------------------------------------------- #
def compressed_attention(
    q, k, v, kernel_size, kernel_stride, block_size, topk, cu_seqlens_q, cu_seqlens_k,
    max_seqlen_q=None, max_seqlen_k=None, sm_scale=None, init_blocks=1, local_blocks=2,
    return_scores=False,
):
    """Output of attention over compressed K/V, and the selected block ids.

    Query at in-sequence position ``t`` sees compressed key ``i`` iff
    ``t >= i*stride + kernel_size - 1``; rows with no visible key give 0.
    ``score[h_kv, t, i]`` is the softmax probability summed over the query heads
    of a KV group.  Follows
    native_sparse_attention/ops/torch/compressed_attention.py:74-194 (mask
    :119-133, attention :135-145, score and top-k :146-193); the number of
    candidate blocks is ``ceil(max_seqlen_q / block_size)`` as in
    ops/triton/compressed_attention.py:1131.
    """
    N, Hq, d = q.shape
    Hkv = k.shape[1]
    dev = q.device
    B = cu_seqlens_q.numel() - 1
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    cu_q, cu_k = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    seqlens_q = [cu_q[b + 1] - cu_q[b] for b in range(B)]
    if max_seqlen_q is None:
        max_seqlen_q = max(seqlens_q)
    num_blocks = math.ceil(max_seqlen_q / block_size)
    outs, idxs, scores = [], [], []
    for b in range(B):
        qs, qe, ks_, ke = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        Lq, Lk = qe - qs, ke - ks_
        kmax = torch.arange(Lk, device=dev) * kernel_stride + kernel_size - 1
        t_all = torch.arange(Lq, device=dev)
        idx_b = torch.empty(Hkv, Lq, min(topk, num_blocks) if topk > 0 else 0, dtype=torch.int32, device=dev)
        sc_b = torch.empty(Hkv, Lq, num_blocks, device=dev) if (topk > 0 and return_scores) else None

        def mask_fn(h, t0, t1):
            return t_all[t0:t1, None] >= kmax[None, :]

        def score_fn(h, t0, t1, p_sum):
            bsc = block_scores_from_key_scores(p_sum, kernel_size, kernel_stride, block_size, num_blocks)
            idx, forced_sc = select_topk_blocks(bsc, t_all[t0:t1] // block_size, topk, init_blocks, local_blocks)
            idx_b[h, t0:t1] = idx
            if sc_b is not None:
                sc_b[h, t0:t1] = forced_sc

        outs.append(_masked_attention(q[qs:qe], k[ks_:ke], v[ks_:ke], mask_fn, sm_scale, score_fn if topk > 0 else None))
        idxs.append(idx_b)
        scores.append(sc_b)
    o = torch.cat(outs, 0).to(q.dtype)
    if topk <= 0:
        return (o, None, None) if return_scores else (o, None)
    topk_idx = torch.cat(idxs, 1)
    if return_scores:
        return o, topk_idx, torch.cat(scores, 1)
    return o, topk_idx


# --------------------------------------------------------------------------- #
# attention over the selected KV blocks (row a4)
# --------------------------------------------------------------------------- #
def topk_sparse_attention(q, k, v, topk_idx, block_size, cu_seqlens, softmax_scale=None):
    """Each query attends to the keys of its selected blocks, causally.

    A block id is used iff ``0 <= id <= t // block_size``; inside a block key
    position ``p`` is visible iff ``p <= t``.  Follows
    native_sparse_attention/ops/torch/topk_sparse_attention.py:19-83 and the
    validity rule of ops/triton/topk_sparse_attention.py:89-93,138.
    """
    N, Hq, d = q.shape
    dev = q.device
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    cu = cu_seqlens.tolist()
    outs = []
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        L = e - s
        nb = math.ceil(L / block_size)
        t_all = torch.arange(L, device=dev)
        idx_seq = topk_idx[:, s:e].long().to(dev)  # [Hkv, L, T]

        def mask_fn(h, t0, t1):
            t = t_all[t0:t1]
            idx = idx_seq[h, t0:t1]
            valid = (idx >= 0) & (idx <= (t // block_size)[:, None])
            sel = torch.zeros(t1 - t0, nb + 1, dtype=torch.bool, device=dev)
            sel.scatter_(1, torch.where(valid, idx, torch.full_like(idx, nb)), True)
            return sel[:, :nb].repeat_interleave(block_size, 1)[:, :L] & (t[:, None] >= t_all[None, :])

        outs.append(_masked_attention(q[s:e], k[s:e], v[s:e], mask_fn, softmax_scale))
    return torch.cat(outs, 0).to(q.dtype)


# --------------------------------------------------------------------------- #
# dense varlen attention (row a8)
# --------------------------------------------------------------------------- #
def flash_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q=None, max_seqlen_k=None,
                           causal=False, sm_scale=None):
    """Dense varlen GQA attention; causal means key ``j`` visible iff ``j <= i`` (top-left aligned).

    Follows native_sparse_attention/ops/triton/flash_attention.py:118-131.
    """
    N, Hq, d = q.shape
    dev = q.device
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    cu_q, cu_k = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    outs = []
    for b in range(len(cu_q) - 1):
        qs, qe, ks_, ke = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        j = torch.arange(ke - ks_, device=dev)

        def mask_fn(h, t0, t1):
            i = torch.arange(t0, t1, device=dev)
            return (i[:, None] >= j[None, :]) if causal else torch.ones(t1 - t0, ke - ks_, dtype=torch.bool, device=dev)

        outs.append(_masked_attention(q[qs:qe], k[ks_:ke], v[ks_:ke], mask_fn, sm_scale))
    return torch.cat(outs, 0).to(q.dtype)


def sliding_window_attention(q, k, v, cu_seqlens, window_size, sm_scale=None):
    """Causal varlen self-attention with a sliding window: query ``i`` sees keys ``i - window_size .. i``.

    The reference delegates this branch to the third-party flash_attn package
    (native_sparse_attention/module/native_sparse_attention.py:213-223, ``causal=True``,
    ``window_size=(window_size, -1)``); this restates flash_attn's published mask semantics for equal query and key
    lengths (key j visible iff i - left <= j <= i).  Pinned by tests/golden/box_window.npz, the output of
    flash_attn.flash_attn_varlen_func itself on a B200 (made by tests/golden/make_golden_on_box.py).
    """
    N, Hq, d = q.shape
    dev = q.device
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    cu = cu_seqlens.tolist()
    outs = []
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        j = torch.arange(e - s, device=dev)

        def mask_fn(h, t0, t1):
            i = torch.arange(t0, t1, device=dev)[:, None]
            return (j[None, :] <= i) & (j[None, :] >= i - window_size)

        outs.append(_masked_attention(q[s:e], k[s:e], v[s:e], mask_fn, sm_scale))
    return torch.cat(outs, 0).to(q.dtype)


# --------------------------------------------------------------------------- #
# single-token (decode) operators (rows a5 - a7)
# --------------------------------------------------------------------------- #
def flash_attention_decode(q, k, v, seqlens, sm_scale=None):
    """One query token per sequence against the first ``seqlens[b]`` cache rows.

    Follows native_sparse_attention/ops/triton/flash_attention_decode.py:103-128.
    """
    B, Hq, d = q.shape
    G = Hq // k.shape[2]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    L = k.shape[1]
    mask = torch.arange(L, device=q.device)[None, :] < seqlens[:, None]
    logits = torch.einsum("bhd,bjhd->bhj", q.float(), k.float().repeat_interleave(G, 2)) * sm_scale
    logits = logits.masked_fill(~mask[:, None, :], float("-inf"))
    p = logits.softmax(-1).nan_to_num(0)
    return torch.einsum("bhj,bjhd->bhd", p, v.float().repeat_interleave(G, 2)).to(q.dtype)


def compressed_attention_decode(q, k, v, seqlens, compress_seqlens, kernel_size, kernel_stride, block_size,
                                topk, init_blocks=1, local_blocks=2, sm_scale=None, return_scores=False):
    """Single-token compressed attention plus block selection.

    ``seqlens`` counts the current token; the query's block is
    ``(seqlens - 1) // block_size`` and the number of candidate blocks is
    ``ceil(max(seqlens) / block_size)``.  An empty compressed cache returns
    zeros and an all-zero index of shape [Hkv, B, 1].  Follows
    native_sparse_attention/ops/torch/compressed_attention_decode.py:65-153.
    """
    B, Hq, d = q.shape
    _, Lc, Hkv, _ = k.shape
    G = Hq // Hkv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    if Lc == 0:
        res = (torch.zeros_like(q), torch.zeros(Hkv, B, 1, dtype=torch.int32, device=q.device))
        return res + (None,) if return_scores else res
    mask = torch.arange(Lc, device=q.device)[None, :] < compress_seqlens[:, None]
    logits = torch.einsum("bhd,bjhd->bhj", q.float(), k.float().repeat_interleave(G, 2)) * sm_scale
    logits = logits.masked_fill(~mask[:, None, :], float("-inf"))
    p = logits.softmax(-1).nan_to_num(0)
    o = torch.einsum("bhj,bjhd->bhd", p, v.float().repeat_interleave(G, 2)).to(q.dtype)
    score = p.reshape(B, Hkv, G, Lc).sum(2).permute(1, 0, 2)  # [Hkv, B, Lc]
    num_blocks = math.ceil(int(seqlens.max()) / block_size)
    bsc = block_scores_from_key_scores(score, kernel_size, kernel_stride, block_size, num_blocks)
    idx, forced = select_topk_blocks(bsc, (seqlens.long() - 1) // block_size, topk, init_blocks, local_blocks)
    if return_scores:
        return o, idx, forced
    return o, idx


def topk_sparse_attention_decode(q, k, v, topk_idx, block_size, seqlens, sm_scale=None):
    """Single-token attention over the selected blocks of a dense cache.

    Block id valid iff ``0 <= id <= (seqlens-1)//block_size``; key position
    valid iff ``< seqlens[b]``.  Follows
    native_sparse_attention/ops/triton/topk_sparse_attention_decode.py:66-122.
    """
    B, Hq, d = q.shape
    _, L, Hkv, _ = k.shape
    G = Hq // Hkv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    nb = math.ceil(L / block_size)
    idx = topk_idx.long()  # [Hkv, B, T]
    valid = (idx >= 0) & (idx <= ((seqlens.long() - 1) // block_size)[None, :, None])
    sel = torch.zeros(Hkv, B, nb + 1, dtype=torch.bool, device=q.device)
    sel.scatter_(2, torch.where(valid, idx, torch.full_like(idx, nb)), True)
    mask = sel[..., :nb].repeat_interleave(block_size, 2)[..., :L]
    mask = mask & (torch.arange(L, device=q.device)[None, None, :] < seqlens[None, :, None])
    mask = mask.permute(1, 0, 2).repeat_interleave(G, 1)  # [B, Hq, L]
    logits = torch.einsum("bhd,bjhd->bhj", q.float(), k.float().repeat_interleave(G, 2)) * sm_scale
    logits = logits.masked_fill(~mask, float("-inf"))
    p = logits.softmax(-1).nan_to_num(0)
    return torch.einsum("bhj,bjhd->bhd", p, v.float().repeat_interleave(G, 2)).to(q.dtype)


# --------------------------------------------------------------------------- #
# comparators
# --------------------------------------------------------------------------- #
def compare_topk_idx(idx_test: torch.Tensor, idx_ref: torch.Tensor, ref_scores: torch.Tensor, tie_tol: float = 1e-3):
    """Tie-aware equality of selected block ids.

    idx_* [H, Q, T] int32 (ascending, -1 padded); ref_scores [H, Q, num_blocks]
    are the reference's block scores with forced blocks at +inf.  A row passes
    when the two id sets are equal, or when every id present in only one of the
    sets has a reference score within ``tie_tol`` of the row's selection
    threshold (the smallest selected reference score).  Returns
    ``(num_bad_rows, num_rows_differing, num_rows)``.
    """
    H, Q, T = idx_ref.shape
    nb = ref_scores.shape[-1]
    a = torch.zeros(H, Q, nb + 1, dtype=torch.bool, device=idx_ref.device)
    b = torch.zeros(H, Q, nb + 1, dtype=torch.bool, device=idx_ref.device)
    a.scatter_(2, torch.where(idx_test >= 0, idx_test.long(), torch.full_like(idx_test, nb).long()), True)
    b.scatter_(2, torch.where(idx_ref >= 0, idx_ref.long(), torch.full_like(idx_ref, nb).long()), True)
    a, b = a[..., :nb], b[..., :nb]
    same_count = a.sum(-1) == b.sum(-1)
    diff = a ^ b
    rows_diff = diff.any(-1)
    inf = torch.full_like(ref_scores, float("inf"))
    thr = torch.where(b, ref_scores, inf).amin(-1, keepdim=True)  # k-th best reference score
    ok_elem = (~diff) | ((ref_scores - thr).abs() <= tie_tol)
    bad_rows = (~ok_elem.all(-1)) | (~same_count)
    return int(bad_rows.sum()), int(rows_diff.sum()), H * Q


def error_stats(test: torch.Tensor, ref: torch.Tensor):
    """(max abs error, mean abs error) in fp32."""
    dlt = (test.float() - ref.float()).abs()
    return float(dlt.max()) if dlt.numel() else 0.0, float(dlt.mean()) if dlt.numel() else 0.0


# --------------------------------------------------------------------------- #
# algorithmic work model (useful FLOPs: unmasked pairs only, 2 GEMMs forward, 5 backward)
# --------------------------------------------------------------------------- #
def visible_pairs_compressed(seqlens, kernel_size, kernel_stride) -> int:
    total = 0
    for L in seqlens:
        M = 0 if L < kernel_size else (L - kernel_size) // kernel_stride + 1
        t = torch.arange(L)
        vis = torch.clamp(torch.div(t - kernel_size + 1, kernel_stride, rounding_mode="floor") + 1, min=0, max=M)
        total += int(vis.sum())
    return total


def visible_pairs_selected(seqlens, block_size, topk) -> int:
    """Pairs per KV head when every query selects min(topk, own_block+1) blocks incl. its own."""
    total = 0
    for L in seqlens:
        t = torch.arange(L)
        bq = t // block_size
        nsel = torch.clamp(bq + 1, max=topk)
        total += int(((nsel - 1) * block_size + t % block_size + 1).sum())
    return total


def useful_flops(seqlens, Hq, Hkv, d, kernel_size, kernel_stride, block_size, topk):
    """dict of forward FLOPs per piece; backward = 2.5x (attention) or 2x (linear compression)."""
    G = Hq // Hkv
    p_cmp = visible_pairs_compressed(seqlens, kernel_size, kernel_stride)
    p_sel = visible_pairs_selected(seqlens, block_size, topk)
    M = sum(0 if L < kernel_size else (L - kernel_size) // kernel_stride + 1 for L in seqlens)
    return {
        "cmp_fwd": 4.0 * d * Hq * p_cmp,
        "sel_fwd": 4.0 * d * G * p_sel * Hkv,
        "lin_fwd": 2.0 * (2.0 * kernel_size * d * d * M * Hkv),
    }


def total_useful_flops(seqlens, Hq, Hkv, d, kernel_size, kernel_stride, block_size, topk, backward=True):
    f = useful_flops(seqlens, Hq, Hkv, d, kernel_size, kernel_stride, block_size, topk)
    fwd = f["cmp_fwd"] + f["sel_fwd"] + f["lin_fwd"]
    if not backward:
        return fwd
    return fwd + 2.5 * (f["cmp_fwd"] + f["sel_fwd"]) + 2.0 * f["lin_fwd"]


def gate_combine(gate, o_cmp, o_sel, o_win):
    """Gated sum of the three branch outputs, gate [n, h, 3], o_* [n, h, d]: the expression of the reference's layer
    (native_sparse_attention/module/native_sparse_attention.py:226-232, infer/nsa_inference.py:146-150) evaluated in fp32.
    Pinned as part of the inference step (tests/golden/box_infer_*.npz: the reference's nsa_infer run on a B200)."""
    g = gate.float()
    out = g[..., 0:1] * o_cmp.float() + g[..., 1:2] * o_sel.float() + g[..., 2:3] * o_win.float()
    return out.to(o_cmp.dtype)


def rope(x, inv_freq, cu_seqlens, step=0, stride=1, attention_scaling=1.0):
    """Rotary embedding of a varlen batch, x [rows, heads, d]: x * cos + rotate_half(x) * sin with rotate_half(x) =
    cat(-x2, x1) (native_sparse_attention/module/rope.py:36-41,204-209); cos/sin of the fp32 angle inv_freq * position,
    times attention_scaling, rounded to x.dtype (:126-155); position t * stride for the t-th token of a sequence when
    step == 0, (seqlen_b + step - 1) * stride for row b when step > 0 (:158-195).  The arithmetic after the table lookup is
    fp32 here (the reference rounds each product to x.dtype).  Pinned by tests/golden/box_rope.npz: outputs of the
    reference's RotaryEmbedding on a B200 (llama3 scaling, prefill / strided / decode positions, bf16 and fp16)."""
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
    if step == 0:
        pos = torch.cat([torch.arange(n) for n in lens]) if lens else torch.zeros(0, dtype=torch.long)
    else:
        pos = torch.tensor([n + step - 1 for n in lens])
    pos = (pos * stride).float().to(x.device)
    ang = inv_freq.float().to(x.device)[None, :] * pos[:, None]
    cos = (ang.cos() * attention_scaling).to(x.dtype).float()
    sin = (ang.sin() * attention_scaling).to(x.dtype).float()
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)


# --------------------------------------------------------------------------- #
# inference step (cache bookkeeping restated as a function of the token history)
# --------------------------------------------------------------------------- #
def nsa_decode_token(q_new, k_hist, v_hist, gate_new, inv_freq, compress_k, compress_v, w_k, w_v, pe, kernel_size,
                     kernel_stride, block_size, topk, init_blocks, local_blocks, window_size, attention_scaling=1.0):
    """Output of one decode step of the reference's NSA inference for ONE sequence, as a function of its history:
    q_new [Hq, d], gate_new [Hq, 3] belong to the newest token; k_hist, v_hist [n, Hkv, d] are the keys/values of all n
    tokens including it, BEFORE rotary embedding.  compress_k / compress_v are the oracle's compress functions.

    What the reference's caches hold at that moment (native_sparse_attention/module/kv_cache.py:233-449, driven by
    infer/nsa_inference.py:77-150 and infer/inference_func.py:27-202) is determined by n alone:
      * its staging buffer is compressed whenever it holds kernel_size tokens and then drops kernel_stride of them, so the
        compressed cache holds the windows [i*stride, i*stride + kernel_size) that fit in n tokens -- the same
        (n - kernel_size) // stride + 1 windows a prefill of n tokens gives -- compressed before rotary embedding, the keys
        then rotated to position i * stride;
      * the selected-block cache holds all n rotated keys and the values; the query is rotated to position n - 1;
      * the sliding-window ring holds the last min(n, window_size) tokens (one fewer than a prefill row sees).
    """
    n = k_hist.shape[0]
    cu = torch.tensor([0, n], dtype=torch.int32)
    ck, cu_c = compress_k(k_hist, w_k, cu, kernel_size, kernel_stride, pe)
    cv, _ = compress_v(v_hist, w_v, cu, kernel_size, kernel_stride, None)
    m = ck.shape[0]
    q_r = rope(q_new[None], inv_freq, torch.tensor([0, n - 1], dtype=torch.int32), 1, 1, attention_scaling)  # position n - 1
    k_r = rope(k_hist, inv_freq, cu, 0, 1, attention_scaling)
    ck_r = rope(ck, inv_freq, cu_c, 0, kernel_stride, attention_scaling) if m > 0 else ck
    lens, clens = torch.tensor([n], dtype=torch.int32), torch.tensor([m], dtype=torch.int32)
    o_cmp, idx = compressed_attention_decode(q_r, ck_r[None], cv[None], lens, clens, kernel_size, kernel_stride, block_size,
                                             topk, init_blocks, local_blocks)
    o_sel = topk_sparse_attention_decode(q_r, k_r[None], v_hist[None], idx, block_size, lens)
    w = min(n, window_size)
    o_win = flash_attention_decode(q_r, k_r[None, n - w:], v_hist[None, n - w:], torch.tensor([w], dtype=torch.int32))
    return gate_combine(gate_new[None], o_cmp, o_sel, o_win)[0]


def nsa_prefill(q, k, v, gate, cu_seqlens, inv_freq, compress_k, compress_v, w_k, w_v, pe, kernel_size, kernel_stride,
                block_size, topk, init_blocks, local_blocks, window_size, attention_scaling=1.0):
    """Prefill step of the reference's NSA inference (infer/nsa_inference.py:77-150 with step == 0): compression before
    rotary embedding, rotation of query / compressed key (positions i * stride) / key, the three branches, the gated sum."""
    ck, cu_c = compress_k(k, w_k, cu_seqlens, kernel_size, kernel_stride, pe)
    cv, _ = compress_v(v, w_v, cu_seqlens, kernel_size, kernel_stride, None)
    q_r = rope(q, inv_freq, cu_seqlens, 0, 1, attention_scaling)
    k_r = rope(k, inv_freq, cu_seqlens, 0, 1, attention_scaling)
    ck_r = rope(ck, inv_freq, cu_c, 0, kernel_stride, attention_scaling)
    o_cmp, idx = compressed_attention(q_r, ck_r, cv, kernel_size, kernel_stride, block_size, topk, cu_seqlens, cu_c,
                                      init_blocks=init_blocks, local_blocks=local_blocks)[:2]
    o_sel = topk_sparse_attention(q_r, k_r, v, idx, block_size, cu_seqlens)
    o_win = sliding_window_attention(q_r, k_r, v, cu_seqlens, window_size)
    return gate_combine(gate, o_cmp, o_sel, o_win)
