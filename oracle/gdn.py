"""CPU oracle (test infrastructure) for Gated Delta Net decode, one token per sequence, state
[batch, 8, 128 (v), 128 (k)] fp32 with k last.

Follows the delta rule as reference/gdn-decode/variants/cuda_bv32_register_resident/kernel.py
states it (:257-326): g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b); per state
row kdot = S k, delta = beta (v - g kdot), S' = g S + delta k^T, out = scale q . S'. Pinned against
the FlashInfer-Bench definition ``gdn_decode_qk4_v8_d128_k_last``
(flashinfer.trace.templates.gdn, fixture tests/golden/gdn_decode_b5.pt).
"""
import math

import torch
import torch.nn.functional as F


def gdn_decode(q, k, v, state, A_log, a, dt_bias, b, scale):
    B, _, hq, K = q.shape
    hv, V = v.shape[2], v.shape[3]
    if scale is None or scale == 0.0:
        scale = 1.0 / math.sqrt(K)
    g = torch.exp(-torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())).reshape(B, hv, 1)
    beta = torch.sigmoid(b.float()).reshape(B, hv, 1)
    qf = q[:, 0].float().repeat_interleave(hv // hq, dim=1)           # [B, hv, K]
    kf = k[:, 0].float().repeat_interleave(hv // k.shape[2], dim=1)
    vf = v[:, 0].float()                                              # [B, hv, V]
    S = state.float() if state is not None else torch.zeros(B, hv, V, K)
    kdot = torch.einsum("bhvk,bhk->bhv", S, kf)
    delta = beta * (vf - g * kdot)
    new_state = g.unsqueeze(-1) * S + delta.unsqueeze(-1) * kf.unsqueeze(2)
    out = scale * torch.einsum("bhvk,bhk->bhv", new_state, qf)
    return out.unsqueeze(1).to(torch.bfloat16), new_state


def gdn_prefill(q, k, v, state, A_log, a, dt_bias, b, cu_seqlens, scale):
    """The decode recurrence applied token by token to every packed sequence (the recurrence that
    reference/gdn-prefill/variants/cuda_graph_v5/kernel.py:1333 evaluates in chunked form); an
    empty sequence leaves a zero new state. Pinned against the FlashInfer-Bench definition
    ``gdn_prefill_qk4_v8_d128_k_last`` (fixture tests/golden/gdn_prefill_s3.pt)."""
    T, hq, K = q.shape
    hv, V = v.shape[1], v.shape[2]
    n = cu_seqlens.numel() - 1
    if scale is None or scale == 0.0:
        scale = 1.0 / math.sqrt(K)
    g = torch.exp(-torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float()))   # [T, hv]
    beta = torch.sigmoid(b.float())
    qf = q.float().repeat_interleave(hv // hq, dim=1)
    kf = k.float().repeat_interleave(hv // k.shape[1], dim=1)
    vf = v.float()
    out = torch.zeros(T, hv, V)
    new_state = torch.zeros(n, hv, V, K)
    for s in range(n):
        t0, t1 = int(cu_seqlens[s]), int(cu_seqlens[s + 1])
        if t1 <= t0:
            continue
        S = state[s].float().clone() if state is not None else torch.zeros(hv, V, K)
        for t in range(t0, t1):
            gt, bt = g[t].view(hv, 1), beta[t].view(hv, 1)
            kdot = torch.einsum("hvk,hk->hv", S, kf[t])
            delta = bt * (vf[t] - gt * kdot)
            S = gt.unsqueeze(-1) * S + delta.unsqueeze(-1) * kf[t].unsqueeze(1)
            out[t] = scale * torch.einsum("hvk,hk->hv", S, qf[t])
        new_state[s] = S
    return out.to(torch.bfloat16), new_state
