"""CPU oracle (TEST INFRASTRUCTURE, never shipped or measured as the product) for the attention
operators: paged GQA decode, paged MLA decode, causal paged MLA prefill, DSA sparse attention.

PyTorch fp32 restatement of the reference plug-ins' arithmetic. All logits in fp32 from exactly
converted bf16 inputs, one final cast to bf16, LSE in base 2 (natural log-sum-exp / ln 2).

Parity pin: the reference repository holds no golden vectors for these operators; this oracle is
pinned against the FlashInfer-Bench operator definitions shipped in flashinfer-python 0.6.11
(``flashinfer.trace.templates``), through the fixtures under ``tests/golden``.
"""
from __future__ import annotations

import math

import torch

_LN2 = math.log(2.0)


def _attend(logits: torch.Tensor, values: torch.Tensor):
    """logits [H, L] fp32 (already scaled), values [L, Dv] fp32 -> (o [H, Dv] fp32, lse2 [H])."""
    lse = torch.logsumexp(logits, dim=-1) / _LN2
    o = torch.softmax(logits, dim=-1) @ values
    return o, lse


def gqa_paged_decode(q, k_cache, v_cache, kv_indptr, kv_indices, sm_scale):
    """Follows reference/gqa-paged-decode-h32-kv8-d128-ps1/variants/
    triton_per_workload_split_max/kernel.py:137-204 (head h reads KV head h // group, :146-149)
    and triton_flash_decode_split_stages4/kernel.py:54-57 (base-2 LSE; empty -> 0 / -inf)."""
    B, HQ, D = q.shape
    _, P, HKV, _ = k_cache.shape
    group = HQ // HKV
    o = torch.zeros(B, HQ, D, dtype=torch.bfloat16)
    lse = torch.full((B, HQ), -float("inf"), dtype=torch.float32)
    qf = q.float()
    for b in range(B):
        s, e = int(kv_indptr[b]), int(kv_indptr[b + 1])
        if e <= s:
            continue
        pages = kv_indices[s:e].long()
        k = k_cache[pages].float().reshape(-1, HKV, D)   # [L, HKV, D]
        v = v_cache[pages].float().reshape(-1, HKV, D)
        qb = qf[b].reshape(HKV, group, D)                 # [HKV, G, D]
        logits = torch.einsum("hgd,lhd->hgl", qb, k) * sm_scale
        l2 = torch.logsumexp(logits, dim=-1) / _LN2
        ob = torch.einsum("hgl,lhd->hgd", torch.softmax(logits, dim=-1), v)
        o[b] = ob.reshape(HQ, D).to(torch.bfloat16)
        lse[b] = l2.reshape(HQ)
    return o, lse


def mla_paged_decode(q_nope, q_pe, ckv_cache, kpe_cache, kv_indptr, kv_indices, sm_scale):
    """Follows reference/mla-paged-decode-h16-ckv512-kpe64-ps1/variants/
    triton_split_kv_2d_reduce_pdl_rw2_brdispatch/kernel.py:152-185 (logit = q_nope.ckv + q_pe.kpe,
    value = ckv) and :182,351-352 (base-2 LSE)."""
    B, H, Dc = q_nope.shape
    Dp = q_pe.shape[-1]
    o = torch.zeros(B, H, Dc, dtype=torch.bfloat16)
    lse = torch.full((B, H), -float("inf"), dtype=torch.float32)
    for b in range(B):
        s, e = int(kv_indptr[b]), int(kv_indptr[b + 1])
        if e <= s:
            continue
        pages = kv_indices[s:e].long()
        kc = ckv_cache[pages].float().reshape(-1, Dc)
        kp = kpe_cache[pages].float().reshape(-1, Dp)
        logits = (q_nope[b].float() @ kc.T + q_pe[b].float() @ kp.T) * sm_scale
        ob, l2 = _attend(logits, kc)
        o[b] = ob.to(torch.bfloat16)
        lse[b] = l2
    return o, lse


def mla_paged_prefill(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices,
                      sm_scale):
    """Follows reference/mla-paged-prefill-causal-h16-ckv512-kpe64-ps1/variants/
    iter6-triton-split-K-grid-pid0-kvsplit/submission_no_cache.py:231-329 (end-aligned causal
    mask: query i sees kv j <= (kv_len - q_len) + i, :244,276,303) and :546-553 (rows that see no
    key keep o = 0, lse = -inf)."""
    TQ, H, Dc = q_nope.shape
    Dp = q_pe.shape[-1]
    o = torch.zeros(TQ, H, Dc, dtype=torch.bfloat16)
    lse = torch.full((TQ, H), -float("inf"), dtype=torch.float32)
    nseq = qo_indptr.shape[0] - 1
    for b in range(nseq):
        qs, qe = int(qo_indptr[b]), int(qo_indptr[b + 1])
        ks, ke = int(kv_indptr[b]), int(kv_indptr[b + 1])
        if qe <= qs or ke <= ks:
            continue
        pages = kv_indices[ks:ke].long()
        kc = ckv_cache[pages].float().reshape(-1, Dc)
        kp = kpe_cache[pages].float().reshape(-1, Dp)
        L = kc.shape[0]
        S = qe - qs
        prefix = L - S
        for c0 in range(0, S, 128):                        # query chunks bound the logits' size
            c1 = min(S, c0 + 128)
            qn = q_nope[qs + c0:qs + c1].float()           # [C, H, Dc]
            qp = q_pe[qs + c0:qs + c1].float()
            hi = min(L, prefix + c1)                       # no query of the chunk sees kv >= hi
            if hi <= 0:
                continue
            logits = (torch.einsum("shd,ld->shl", qn, kc[:hi])
                      + torch.einsum("shd,ld->shl", qp, kp[:hi])) * sm_scale
            pos = torch.arange(c0, c1).unsqueeze(1) + prefix   # last visible kv index per query
            visible = torch.arange(hi).unsqueeze(0) <= pos     # [C, hi]
            logits = logits.masked_fill(~visible.unsqueeze(1), -float("inf"))
            has_any = visible.any(dim=1)
            l2 = torch.logsumexp(logits, dim=-1) / _LN2
            p = torch.nan_to_num(torch.softmax(logits, dim=-1), nan=0.0)
            ob = torch.einsum("shl,ld->shd", p, kc[:hi])
            idx = torch.nonzero(has_any).squeeze(1)
            o[qs + c0 + idx] = ob[idx].to(torch.bfloat16)
            lse[qs + c0 + idx] = l2[idx]
    return o, lse


def dsa_sparse_attention(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale):
    """Follows reference/dsa-sparse-attention/variants/pure_triton/kernel.py:36-101 (keys are the
    rows sparse_indices[t] of the flattened caches, -1 ignored, :44-57; lse = (m + ln l) * log2 e,
    :98-100) and :154-155 (cache flattening)."""
    T, H, Dc = q_nope.shape
    Dp = q_pe.shape[-1]
    kc_all = ckv_cache.reshape(-1, Dc)
    kp_all = kpe_cache.reshape(-1, Dp)
    o = torch.zeros(T, H, Dc, dtype=torch.bfloat16)
    lse = torch.full((T, H), -float("inf"), dtype=torch.float32)
    for t in range(T):
        idx = sparse_indices[t]
        idx = idx[idx != -1].long()
        if idx.numel() == 0:
            continue
        kc = kc_all[idx].float()
        kp = kp_all[idx].float()
        logits = (q_nope[t].float() @ kc.T + q_pe[t].float() @ kp.T) * sm_scale
        ob, l2 = _attend(logits, kc)
        o[t] = ob.to(torch.bfloat16)
        lse[t] = l2
    return o, lse
