"""Paged GQA decode (32 query heads, 8 KV heads, head_dim 128, bf16).

Same signature and return convention as the reference plug-in
``run(q, k_cache, v_cache, kv_indptr, kv_indices, sm_scale) -> (o, lse)``
(reference/gqa-paged-decode-h32-kv8-d128-ps1/variants/triton_pdl_grid_dispatch/kernel.py:420-532).
"""
import torch

from . import _cabi


@torch.no_grad()
def run(q, k_cache, v_cache, kv_indptr, kv_indices, sm_scale):
    if q.dim() != 3 or q.shape[1] != 32 or q.shape[2] != 128:
        raise _cabi.Ako4xError("gqa_decode: q must be [batch, 32, 128]")
    if k_cache.dim() != 4 or k_cache.shape[2] != 8 or k_cache.shape[3] != 128 \
            or v_cache.shape != k_cache.shape:
        raise _cabi.Ako4xError("gqa_decode: caches must be [pages, page_size, 8, 128]")
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise _cabi.Ako4xError("gqa_decode: bf16 tensors expected")
    if kv_indptr.dtype != torch.int32 or kv_indices.dtype != torch.int32:
        raise _cabi.Ako4xError("gqa_decode: kv_indptr / kv_indices must be int32")
    batch = q.shape[0]
    if kv_indptr.numel() != batch + 1:
        raise _cabi.Ako4xError("gqa_decode: kv_indptr must have batch + 1 entries")
    page_size = k_cache.shape[1]
    n_idx = kv_indices.numel()
    L = _cabi.lib()
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.empty((batch, 32), dtype=torch.float32, device=q.device)
    ws_bytes = L.ako4x_gqa_paged_decode_workspace_bytes(batch, n_idx, page_size)
    ws = _cabi.workspace(ws_bytes, q.device)
    qc = q.contiguous()   # kept alive until the launch is enqueued
    st = L.ako4x_gqa_paged_decode(
        _cabi.ptr(qc), _cabi.ptr(k_cache), _cabi.ptr(v_cache), _cabi.ptr(kv_indptr),
        _cabi.ptr(kv_indices), float(sm_scale), _cabi.ptr(o), _cabi.ptr(lse), batch, n_idx,
        page_size, _cabi.ptr(ws), ws_bytes, _cabi.stream())
    del qc
    _cabi.check(st, "ako4x_gqa_paged_decode")
    return o, lse
