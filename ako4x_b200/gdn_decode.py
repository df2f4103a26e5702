"""Gated Delta Net decode (4 q/k heads, 8 v heads, head size 128, k-last fp32 state).

Same signature as the reference plug-in ``run(q, k, v, state, A_log, a, dt_bias, b, scale)``
(reference/gdn-decode/variants/cuda_bv32_register_resident/kernel.py:456-523): returns
``(output bf16 [B, 1, 8, 128], new_state fp32 [B, 8, 128, 128])``; ``state=None`` means zeros,
``scale`` of None or 0 means 1/sqrt(128).
"""
import math

import torch

from . import _cabi


@torch.no_grad()
def run(q, k, v, state, A_log, a, dt_bias, b, scale):
    if q.dim() != 4 or tuple(q.shape[1:]) != (1, 4, 128) or tuple(k.shape) != tuple(q.shape):
        raise _cabi.Ako4xError("gdn_decode: q and k must be [batch, 1, 4, 128]")
    B = q.shape[0]
    if tuple(v.shape) != (B, 1, 8, 128):
        raise _cabi.Ako4xError("gdn_decode: v must be [batch, 1, 8, 128]")
    if any(t.dtype != torch.bfloat16 for t in (q, k, v, a, b)):
        raise _cabi.Ako4xError("gdn_decode: q, k, v, a, b must be bf16")
    if A_log.numel() != 8 or dt_bias.numel() != 8 or a.numel() != B * 8 or b.numel() != B * 8:
        raise _cabi.Ako4xError("gdn_decode: A_log, dt_bias must have 8 elements, a and b batch * 8")
    if state is not None and (tuple(state.shape) != (B, 8, 128, 128) or state.dtype != torch.float32):
        raise _cabi.Ako4xError("gdn_decode: state must be fp32 [batch, 8, 128, 128]")
    if scale is None or scale == 0.0:
        scale = 1.0 / math.sqrt(128.0)
    qc, kc, vc, ac, bc = q.contiguous(), k.contiguous(), v.contiguous(), a.contiguous(), b.contiguous()
    sc = state.contiguous() if state is not None else None
    Ac, dc = A_log.float().contiguous(), dt_bias.float().contiguous()
    out = torch.empty((B, 1, 8, 128), dtype=torch.bfloat16, device=q.device)
    new_state = torch.empty((B, 8, 128, 128), dtype=torch.float32, device=q.device)
    st = _cabi.lib().ako4x_gdn_decode(_cabi.ptr(qc), _cabi.ptr(kc), _cabi.ptr(vc),
                                      _cabi.ptr(sc) if sc is not None else None, _cabi.ptr(Ac), _cabi.ptr(ac),
                                      _cabi.ptr(dc), _cabi.ptr(bc), float(scale), _cabi.ptr(out),
                                      _cabi.ptr(new_state), B, _cabi.stream())
    _cabi.check(st, "ako4x_gdn_decode")
    return out, new_state
