"""DSA FP8 top-k indexer (64 index heads, dim 128, 64-token pages, top-2048).

Same signature and return convention as the reference plug-in
``run(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table) -> (topk_indices,)``
(reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py:569-655). The cache may arrive as
any dtype/shape whose first dimension is the page count and which holds 8448 bytes per page.

Selection ranks the fp32 scores exactly (ties: lower token position); each row lists its selected
global cache slots in ascending token position, then -1.
"""
import torch

from . import _cabi

PAGE_BYTES = 8448
TOPK = 2048


def _check(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table):
    rows = q_index_fp8.shape[0]
    if q_index_fp8.shape[1:] != (64, 128) or q_index_fp8.element_size() != 1:
        raise _cabi.Ako4xError("dsa_indexer: q_index_fp8 must be e4m3 [rows, 64, 128]")
    npages = k_index_cache_fp8.shape[0]
    if k_index_cache_fp8.numel() * k_index_cache_fp8.element_size() != npages * PAGE_BYTES:
        raise _cabi.Ako4xError("dsa_indexer: cache must hold 8448 bytes per page")
    if weights.dtype != torch.float32 or weights.shape != (rows, 64):
        raise _cabi.Ako4xError("dsa_indexer: weights must be fp32 [rows, 64]")
    if seq_lens.dtype != torch.int32 or block_table.dtype != torch.int32 \
            or seq_lens.numel() != rows or block_table.shape[0] != rows:
        raise _cabi.Ako4xError("dsa_indexer: seq_lens int32 [rows], block_table int32 [rows, pages]")
    return rows, npages, block_table.shape[1]


@torch.no_grad()
def run(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table):
    rows, npages, max_pages = _check(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table)
    L = _cabi.lib()
    dev = q_index_fp8.device
    out = torch.empty((rows, TOPK), dtype=torch.int32, device=dev)
    ws_bytes = L.ako4x_dsa_topk_indexer_workspace_bytes(rows, max_pages)
    ws = _cabi.workspace(ws_bytes, dev)
    keep = [t.contiguous() for t in (q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table)]
    st = L.ako4x_dsa_topk_indexer(
        *[_cabi.ptr(t) for t in keep], _cabi.ptr(out), rows, max_pages, npages,
        _cabi.ptr(ws), ws_bytes, _cabi.stream())
    del keep   # contiguous copies live until the launch has been enqueued
    _cabi.check(st, "ako4x_dsa_topk_indexer")
    return (out,)


@torch.no_grad()
def index_scores(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table):
    """fp32 scores [rows, max_pages*64] (entries at t >= seq_len are -inf or unwritten pages)."""
    rows, npages, max_pages = _check(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table)
    scores = torch.full((rows, max_pages * 64), float("-inf"), dtype=torch.float32,
                        device=q_index_fp8.device)
    keep = [t.contiguous() for t in (q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table)]
    st = _cabi.lib().ako4x_dsa_index_scores(
        *[_cabi.ptr(t) for t in keep], _cabi.ptr(scores), rows, max_pages, npages, _cabi.stream())
    del keep
    _cabi.check(st, "ako4x_dsa_index_scores")
    return scores


@torch.no_grad()
def topk_select(scores, seq_lens, block_table):
    """Exact top-2048 selection on given fp32 scores [rows, max_pages*64]."""
    rows, max_pages = block_table.shape
    if scores.dtype != torch.float32 or scores.shape != (rows, max_pages * 64):
        raise _cabi.Ako4xError("topk_select: scores must be fp32 [rows, max_pages*64]")
    out = torch.empty((rows, TOPK), dtype=torch.int32, device=scores.device)
    keep = [t.contiguous() for t in (scores, seq_lens, block_table)]
    st = _cabi.lib().ako4x_dsa_topk_select(
        *[_cabi.ptr(t) for t in keep], _cabi.ptr(out), rows, max_pages, _cabi.stream())
    del keep
    _cabi.check(st, "ako4x_dsa_topk_select")
    return out


@torch.no_grad()
def run_with_attention(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, q_nope, q_pe, ckv_cache,
                       kpe_cache, sm_scale):
    """Indexer followed by sparse MLA attention in one call, the top-k list staying on the device
    (the pair of reference plug-ins dsa-topk-indexer / dsa-sparse-attention run back to back).
    Returns (o, lse, topk_indices)."""
    from .mla_decode import check_mla_inputs
    rows, npages, max_pages = _check(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table)
    check_mla_inputs("dsa_indexer_attention", q_nope, q_pe, ckv_cache, kpe_cache)
    if q_nope.shape[0] != rows or ckv_cache.shape[0] != npages or ckv_cache.shape[1] != 64:
        raise _cabi.Ako4xError("dsa_indexer_attention: one query row per indexer row, caches of [pages, 64, .]")
    L = _cabi.lib()
    dev = q_index_fp8.device
    topk = torch.empty((rows, TOPK), dtype=torch.int32, device=dev)
    o = torch.empty(q_nope.shape, dtype=q_nope.dtype, device=dev)
    lse = torch.empty((rows, 16), dtype=torch.float32, device=dev)
    ws_bytes = L.ako4x_dsa_indexer_attention_workspace_bytes(rows, max_pages)
    ws = _cabi.workspace(ws_bytes, dev)
    keep = [t.contiguous() for t in (q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, q_nope, q_pe)]
    st = L.ako4x_dsa_indexer_attention(
        *[_cabi.ptr(t) for t in keep], _cabi.ptr(ckv_cache), _cabi.ptr(kpe_cache), float(sm_scale),
        _cabi.ptr(topk), _cabi.ptr(o), _cabi.ptr(lse), rows, max_pages, npages, _cabi.ptr(ws), ws_bytes,
        _cabi.stream())
    del keep
    _cabi.check(st, "ako4x_dsa_indexer_attention")
    return o, lse, topk
