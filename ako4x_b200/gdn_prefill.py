"""Gated Delta Net prefill (4 q/k heads, 8 v heads, head size 128, k-last fp32 state), sequences
packed along the token axis.

Same signature as the reference plug-in ``run(q, k, v, state, A_log, a, dt_bias, b, cu_seqlens,
scale)`` (reference/gdn-prefill/variants/cuda_graph_v5/kernel.py:1333): returns ``(output bf16
[T, 8, 128], new_state fp32 [num_seqs, 8, 128, 128])``; ``state=None`` means zeros, ``scale`` of
None or 0 means 1/sqrt(128).
"""
import math

import torch

from . import _cabi


@torch.no_grad()
def run(q, k, v, state, A_log, a, dt_bias, b, cu_seqlens, scale, _chunked=True):
    if q.dim() != 3 or tuple(q.shape[1:]) != (4, 128) or tuple(k.shape) != tuple(q.shape):
        raise _cabi.Ako4xError("gdn_prefill: q and k must be [tokens, 4, 128]")
    T = q.shape[0]
    if tuple(v.shape) != (T, 8, 128):
        raise _cabi.Ako4xError("gdn_prefill: v must be [tokens, 8, 128]")
    if any(t.dtype != torch.bfloat16 for t in (q, k, v, a, b)):
        raise _cabi.Ako4xError("gdn_prefill: q, k, v, a, b must be bf16")
    if A_log.numel() != 8 or dt_bias.numel() != 8 or a.numel() != T * 8 or b.numel() != T * 8:
        raise _cabi.Ako4xError("gdn_prefill: A_log, dt_bias must have 8 elements, a and b tokens * 8")
    n = cu_seqlens.numel() - 1
    if n < 0:
        raise _cabi.Ako4xError("gdn_prefill: cu_seqlens must have num_seqs + 1 entries")
    if state is not None and (tuple(state.shape) != (n, 8, 128, 128) or state.dtype != torch.float32):
        raise _cabi.Ako4xError("gdn_prefill: state must be fp32 [num_seqs, 8, 128, 128]")
    if scale is None or scale == 0.0:
        scale = 1.0 / math.sqrt(128.0)
    qc, kc, vc, ac, bc = q.contiguous(), k.contiguous(), v.contiguous(), a.contiguous(), b.contiguous()
    sc = state.contiguous() if state is not None else None
    Ac, dc = A_log.float().contiguous(), dt_bias.float().contiguous()
    cu = cu_seqlens.to(torch.int64).contiguous()
    # tokens outside every sequence keep a defined value
    out = torch.zeros((T, 8, 128), dtype=torch.bfloat16, device=q.device)
    new_state = torch.empty((n, 8, 128, 128), dtype=torch.float32, device=q.device)
    lib = _cabi.lib()
    # the chunked form needs room for its per-chunk tables; _chunked=False runs token by token
    ws_bytes = lib.ako4x_gdn_prefill_workspace_bytes(T, n) if _chunked else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
    st = lib.ako4x_gdn_prefill(_cabi.ptr(qc), _cabi.ptr(kc), _cabi.ptr(vc),
                               _cabi.ptr(sc) if sc is not None else None, _cabi.ptr(Ac), _cabi.ptr(ac),
                               _cabi.ptr(dc), _cabi.ptr(bc), _cabi.ptr(cu), float(scale), _cabi.ptr(out),
                               _cabi.ptr(new_state), T, n, _cabi.ptr(ws) if ws is not None else None, ws_bytes,
                               _cabi.stream())
    _cabi.check(st, "ako4x_gdn_prefill")
    return out, new_state
