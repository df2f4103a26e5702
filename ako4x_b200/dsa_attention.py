"""DSA sparse MLA attention (16 heads, ckv 512, kpe 64, bf16; keys chosen per token by index).

Same signature and return convention as the reference plug-in
``run(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale) -> (o, lse)``
(reference/dsa-sparse-attention/variants/hybrid_pdl_v2/kernel.py:557-626).
"""
import torch

from . import _cabi
from .mla_decode import check_mla_inputs


@torch.no_grad()
def run(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale):
    check_mla_inputs("dsa_attention", q_nope, q_pe, ckv_cache, kpe_cache)
    tokens = q_nope.shape[0]
    if sparse_indices.dtype != torch.int32 or sparse_indices.dim() != 2 \
            or sparse_indices.shape[0] != tokens:
        raise _cabi.Ako4xError("dsa_attention: sparse_indices must be int32 [tokens, topk]")
    topk = sparse_indices.shape[1]
    rows = ckv_cache.shape[0] * ckv_cache.shape[1]
    L = _cabi.lib()
    o = torch.empty(q_nope.shape, dtype=q_nope.dtype, device=q_nope.device)
    lse = torch.empty((tokens, 16), dtype=torch.float32, device=q_nope.device)
    ws_bytes = L.ako4x_dsa_sparse_attention_workspace_bytes(tokens, topk)
    ws = _cabi.workspace(ws_bytes, q_nope.device)
    qn, qp, idx = q_nope.contiguous(), q_pe.contiguous(), sparse_indices.contiguous()
    st = L.ako4x_dsa_sparse_attention(
        _cabi.ptr(qn), _cabi.ptr(qp), _cabi.ptr(ckv_cache),
        _cabi.ptr(kpe_cache), _cabi.ptr(idx), float(sm_scale),
        _cabi.ptr(o), _cabi.ptr(lse), tokens, topk, rows, _cabi.ptr(ws), ws_bytes, _cabi.stream())
    del qn, qp, idx
    _cabi.check(st, "ako4x_dsa_sparse_attention")
    return o, lse
