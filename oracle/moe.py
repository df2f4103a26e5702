"""CPU oracle (test infrastructure) for the FP8 block-scale MoE with DeepSeek-V3 routing.

Routing follows reference/moe-fp8-block-scale/variants/fused_routing_v2/kernel.py:350-391:
s = sigmoid(logit); sb = s + bias; group score = sum of the two largest sb in each of 8 groups of
32; keep the 4 best groups; pick the 8 best experts by sb among them; weight = s_e / sum_sel(s)
* routed_scaling_factor, normalised over all 8 selected experts whether local or not
(:396-397). Ties go to the lower index (stable sort). Experts follow :316-330 (block-scale
dequantisation: value x scale per 128 columns of the activations, per 128x128 block of the
weights), :491-495 (h = silu(g[2048:]) * g[:2048]) and :453-474 (out[t] += weight * y).
Layouts: hidden_states_scale is [56, tokens]; weight scales [E, N/128, K/128]
(reference/moe-fp8-block-scale-ds-routing-topk8-ng8-kg4-e32-h7168-i2048/variants/
iter1-trtllm-turnkey-seed/kernel.py:56-65). The intermediate is kept in fp32 (no re-quantisation),
contributions are accumulated in fp32 (or fp64 with ``accum_dtype``) and rounded to bf16 once.

Pinned against flashinfer.trace.templates.moe (fixtures under tests/golden).
"""
import torch

N_GROUP = 8
TOPK_GROUP = 4
TOP_K = 8
BLOCK = 128


def ds_routing(routing_logits, routing_bias, routed_scaling_factor):
    """-> (topk_ids int32 [T,8] ascending expert id, topk_weights fp32 [T,8])."""
    logits = routing_logits.float()
    T, E = logits.shape
    s = torch.sigmoid(logits)
    sb = s + routing_bias.float().reshape(1, E)
    gs = E // N_GROUP
    grouped = sb.view(T, N_GROUP, gs)
    top2 = torch.sort(grouped, dim=2, descending=True, stable=True).values[:, :, :2]
    group_score = top2.sum(dim=2)
    gorder = torch.sort(group_score, dim=1, descending=True, stable=True).indices[:, :TOPK_GROUP]
    gmask = torch.zeros(T, N_GROUP, dtype=torch.bool)
    gmask.scatter_(1, gorder, True)
    emask = gmask.unsqueeze(2).expand(T, N_GROUP, gs).reshape(T, E)
    pruned = sb.masked_fill(~emask, -float("inf"))
    ids = torch.sort(pruned, dim=1, descending=True, stable=True).indices[:, :TOP_K]
    ids = torch.sort(ids, dim=1).values
    sel = s.gather(1, ids)
    w = sel / (sel.sum(dim=1, keepdim=True) + 1e-20) * routed_scaling_factor
    return ids.to(torch.int32), w


def _dequant_weight(w_fp8, scale):
    s = scale.float().repeat_interleave(BLOCK, dim=-2).repeat_interleave(BLOCK, dim=-1)
    return w_fp8.float() * s


def moe_fp8_block_scale(routing_logits, routing_bias, hidden_states, hidden_states_scale,
                        gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale,
                        local_expert_offset, routed_scaling_factor, accum_dtype=torch.float32):
    T, H = hidden_states.shape
    E_local, two_i, _ = gemm1_weights.shape
    I = two_i // 2
    ids, w = ds_routing(routing_logits, routing_bias, routed_scaling_factor)
    a_scale = hidden_states_scale.float().t().contiguous()            # [T, H/128]
    a = hidden_states.float() * a_scale.repeat_interleave(BLOCK, dim=1)
    out = torch.zeros(T, H, dtype=accum_dtype)
    off = int(local_expert_offset)
    for le in range(E_local):
        ge = off + le
        hit = ids == ge                                               # [T, 8]
        tok = torch.nonzero(hit.any(dim=1)).squeeze(1)
        if tok.numel() == 0:
            continue
        w13 = _dequant_weight(gemm1_weights[le], gemm1_weights_scale[le])
        w2 = _dequant_weight(gemm2_weights[le], gemm2_weights_scale[le])
        g = a[tok] @ w13.t()
        x1, x2 = g[:, :I], g[:, I:]
        h = (x2 / (1.0 + torch.exp(-x2))) * x1
        y = h @ w2.t()
        we = (w[tok] * hit[tok].float()).sum(dim=1, keepdim=True)
        out.index_add_(0, tok, (y * we).to(accum_dtype))
    return out.to(torch.bfloat16)
