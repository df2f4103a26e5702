"""Causal paged MLA prefill (16 heads, ckv 512, kpe 64, bf16, ragged batch).

Same signature and return convention as the reference plug-in
``run(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, sm_scale) -> (o, lse)``
(reference/mla-paged-prefill-causal-h16-ckv512-kpe64-ps1/variants/
iter6-triton-split-K-grid-pid0-kvsplit/submission_no_cache.py:537-692). No host read of the
indptr arrays takes place: the launch geometry depends on shapes only.
"""
import torch

from . import _cabi
from .mla_decode import check_mla_inputs


@torch.no_grad()
def run(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, sm_scale):
    check_mla_inputs("mla_prefill", q_nope, q_pe, ckv_cache, kpe_cache)
    for t in (qo_indptr, kv_indptr, kv_indices):
        if t.dtype != torch.int32:
            raise _cabi.Ako4xError("mla_prefill: indptr / indices must be int32")
    if qo_indptr.numel() != kv_indptr.numel():
        raise _cabi.Ako4xError("mla_prefill: qo_indptr and kv_indptr must have the same length")
    total_q = q_nope.shape[0]
    batch = qo_indptr.numel() - 1
    page_size = ckv_cache.shape[1]
    n_idx = kv_indices.numel()
    L = _cabi.lib()
    o = torch.empty(q_nope.shape, dtype=q_nope.dtype, device=q_nope.device)
    lse = torch.empty((total_q, 16), dtype=torch.float32, device=q_nope.device)
    ws_bytes = L.ako4x_mla_paged_prefill_workspace_bytes(total_q, batch, n_idx, page_size)
    ws = _cabi.workspace(ws_bytes, q_nope.device)
    qn, qp = q_nope.contiguous(), q_pe.contiguous()   # kept alive until the launch is enqueued
    st = L.ako4x_mla_paged_prefill(
        _cabi.ptr(qn), _cabi.ptr(qp), _cabi.ptr(ckv_cache),
        _cabi.ptr(kpe_cache), _cabi.ptr(qo_indptr), _cabi.ptr(kv_indptr), _cabi.ptr(kv_indices),
        float(sm_scale), _cabi.ptr(o), _cabi.ptr(lse), total_q, batch, n_idx, page_size,
        _cabi.ptr(ws), ws_bytes, _cabi.stream())
    del qn, qp
    _cabi.check(st, "ako4x_mla_paged_prefill")
    return o, lse
