"""Paged MLA decode (16 heads, ckv 512, kpe 64, bf16).

Same signature and return convention as the reference plug-in
``run(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, sm_scale) -> (o, lse)``
(reference/mla-paged-decode-h16-ckv512-kpe64-ps1/variants/triton_split_kv_2d_reduce_pdl_rw2/kernel.py:369-435).
"""
import torch

from . import _cabi


def check_mla_inputs(op, q_nope, q_pe, ckv_cache, kpe_cache):
    if q_nope.dim() != 3 or q_nope.shape[1:] != (16, 512) or q_pe.shape != (q_nope.shape[0], 16, 64):
        raise _cabi.Ako4xError(f"{op}: q_nope must be [n,16,512] and q_pe [n,16,64]")
    if ckv_cache.dim() != 3 or ckv_cache.shape[2] != 512 or kpe_cache.shape != (*ckv_cache.shape[:2], 64):
        raise _cabi.Ako4xError(f"{op}: caches must be [pages,page_size,512] and [pages,page_size,64]")
    for t in (q_nope, q_pe, ckv_cache, kpe_cache):
        if t.dtype != torch.bfloat16:
            raise _cabi.Ako4xError(f"{op}: bf16 tensors expected")


@torch.no_grad()
def run(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, sm_scale):
    check_mla_inputs("mla_decode", q_nope, q_pe, ckv_cache, kpe_cache)
    if kv_indptr.dtype != torch.int32 or kv_indices.dtype != torch.int32:
        raise _cabi.Ako4xError("mla_decode: kv_indptr / kv_indices must be int32")
    batch = q_nope.shape[0]
    if kv_indptr.numel() != batch + 1:
        raise _cabi.Ako4xError("mla_decode: kv_indptr must have batch + 1 entries")
    page_size = ckv_cache.shape[1]
    n_idx = kv_indices.numel()
    L = _cabi.lib()
    o = torch.empty(q_nope.shape, dtype=q_nope.dtype, device=q_nope.device)
    lse = torch.empty((batch, 16), dtype=torch.float32, device=q_nope.device)
    ws_bytes = L.ako4x_mla_paged_decode_workspace_bytes(batch, n_idx, page_size)
    ws = _cabi.workspace(ws_bytes, q_nope.device)
    qn, qp = q_nope.contiguous(), q_pe.contiguous()   # kept alive until the launch is enqueued
    st = L.ako4x_mla_paged_decode(
        _cabi.ptr(qn), _cabi.ptr(qp), _cabi.ptr(ckv_cache),
        _cabi.ptr(kpe_cache), _cabi.ptr(kv_indptr), _cabi.ptr(kv_indices), float(sm_scale),
        _cabi.ptr(o), _cabi.ptr(lse), batch, n_idx, page_size, _cabi.ptr(ws), ws_bytes,
        _cabi.stream())
    del qn, qp
    _cabi.check(st, "ako4x_mla_paged_decode")
    return o, lse
