"""FP8 block-scale MoE with DeepSeek-V3 grouped routing (256 experts, top-8 of the 4 best of 8
groups; hidden 7168, intermediate 2048; the local experts of one expert-parallel rank).

Same signature and return convention as the reference plug-in
``run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
routed_scaling_factor) -> out``
(reference/moe-fp8-block-scale/variants/fused_routing_v2/kernel.py:509-667).
"""
import torch

from . import _cabi

HIDDEN = 7168
INTER = 2048
NUM_EXPERTS = 256


def _scalar(v):
    return v.item() if torch.is_tensor(v) else v


@torch.no_grad()
def run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
        routed_scaling_factor, _check_status=False):
    tokens = hidden_states.shape[0]
    n_local = gemm1_weights.shape[0]
    if routing_logits.shape != (tokens, NUM_EXPERTS) or routing_logits.dtype != torch.float32:
        raise _cabi.Ako4xError("moe: routing_logits must be fp32 [tokens, 256]")
    if routing_bias.numel() != NUM_EXPERTS or routing_bias.dtype not in (torch.float32, torch.bfloat16):
        raise _cabi.Ako4xError("moe: routing_bias must be fp32 or bf16 [256]")
    if hidden_states.shape != (tokens, HIDDEN) or hidden_states.element_size() != 1:
        raise _cabi.Ako4xError("moe: hidden_states must be e4m3 [tokens, 7168]")
    if hidden_states_scale.shape != (HIDDEN // 128, tokens) or hidden_states_scale.dtype != torch.float32:
        raise _cabi.Ako4xError("moe: hidden_states_scale must be fp32 [56, tokens]")
    if gemm1_weights.shape != (n_local, 2 * INTER, HIDDEN) or gemm1_weights.element_size() != 1:
        raise _cabi.Ako4xError("moe: gemm1_weights must be e4m3 [E, 4096, 7168]")
    if gemm1_weights_scale.shape != (n_local, 2 * INTER // 128, HIDDEN // 128):
        raise _cabi.Ako4xError("moe: gemm1_weights_scale must be fp32 [E, 32, 56]")
    if gemm2_weights.shape != (n_local, HIDDEN, INTER) or gemm2_weights.element_size() != 1:
        raise _cabi.Ako4xError("moe: gemm2_weights must be e4m3 [E, 7168, 2048]")
    if gemm2_weights_scale.shape != (n_local, HIDDEN // 128, INTER // 128):
        raise _cabi.Ako4xError("moe: gemm2_weights_scale must be fp32 [E, 56, 16]")
    dev = hidden_states.device
    L = _cabi.lib()
    out = torch.empty((tokens, HIDDEN), dtype=torch.bfloat16, device=dev)
    ws_bytes = L.ako4x_moe_fp8_block_scale_workspace_bytes(tokens, n_local)
    ws = _cabi.workspace(ws_bytes, dev)
    # Contiguous copies (if any were needed) stay bound until the launch has been enqueued: a
    # temporary freed earlier could be handed to the next copy on the same stream.
    lg, rb, x, xs = (routing_logits.contiguous(), routing_bias.contiguous(),
                     hidden_states.contiguous(), hidden_states_scale.contiguous())
    s13, s2 = gemm1_weights_scale.contiguous(), gemm2_weights_scale.contiguous()
    st = L.ako4x_moe_fp8_block_scale(
        _cabi.ptr(lg), _cabi.ptr(rb), 1 if routing_bias.dtype == torch.bfloat16 else 0,
        _cabi.ptr(x), _cabi.ptr(xs), _cabi.ptr(gemm1_weights), _cabi.ptr(s13),
        _cabi.ptr(gemm2_weights), _cabi.ptr(s2), int(_scalar(local_expert_offset)),
        float(_scalar(routed_scaling_factor)), _cabi.ptr(out), tokens, n_local, _cabi.ptr(ws),
        ws_bytes, _cabi.stream())
    del lg, rb, x, xs, s13, s2
    _cabi.check(st, "ako4x_moe_fp8_block_scale")
    if _check_status:
        off = L.ako4x_moe_fp8_block_scale_status_offset(tokens)
        code = int(ws[off:off + 4].view(torch.int32).item())   # synchronises: tests only
        if code != 0:
            raise _cabi.Ako4xError(f"moe: a bounded device wait gave up (status {code})")
    return out


def run_checked(*args):
    """``run`` followed by a read of the device status word (synchronises the stream)."""
    return run(*args, _check_status=True)


@torch.no_grad()
def ep_combine(rows, pos):
    """Expert-parallel combine: out[t] = bf16(sum over ranks, ascending, of rows[pos[t, g]])."""
    tokens, world = pos.shape
    cols = rows.shape[1]
    if rows.dtype != torch.bfloat16 or pos.dtype != torch.int32:
        raise _cabi.Ako4xError("ep_combine: rows bf16 [n, cols], pos int32 [tokens, world]")
    out = torch.empty((tokens, cols), dtype=torch.bfloat16, device=pos.device)
    rows_c, pos_c = rows.contiguous(), pos.contiguous()
    st = _cabi.lib().ako4x_moe_ep_combine(
        _cabi.ptr(rows_c) if rows.numel() else None, _cabi.ptr(pos_c),
        _cabi.ptr(out), tokens, world, cols, _cabi.stream())
    del rows_c, pos_c
    _cabi.check(st, "ako4x_moe_ep_combine")
    return out


@torch.no_grad()
def ds_routing(routing_logits, routing_bias, routed_scaling_factor):
    """The routing stage alone: (topk_ids int32 [tokens,8] ascending, topk_weights fp32 [tokens,8])."""
    tokens = routing_logits.shape[0]
    dev = routing_logits.device
    ids = torch.empty((tokens, 8), dtype=torch.int32, device=dev)
    w = torch.empty((tokens, 8), dtype=torch.float32, device=dev)
    lg, rb = routing_logits.contiguous(), routing_bias.contiguous()
    st = _cabi.lib().ako4x_moe_ds_routing(
        _cabi.ptr(lg), _cabi.ptr(rb),
        1 if routing_bias.dtype == torch.bfloat16 else 0, float(_scalar(routed_scaling_factor)),
        _cabi.ptr(ids), _cabi.ptr(w), tokens, _cabi.stream())
    del lg, rb
    _cabi.check(st, "ako4x_moe_ds_routing")
    return ids, w
