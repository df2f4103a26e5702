"""Expert-parallel FP8 MoE: one process per GPU, rank r owns experts [32r, 32r+32) (with 8 groups
of 32 experts that is exactly routing group r, so a token reaches at most 4 ranks).

The reference has no distributed path; this module is the multi-GPU form of the operator in
``moe.py``. Per step every rank
  1. routes its own tokens (CUDA routing kernel),
  2. sends ONE copy of a token's e4m3 row, its 56 scales and its 256 router logits to each rank
     that owns at least one of its experts (NCCL all-to-all, rows ordered by destination then
     token, so the layout is deterministic),
  3. runs the single-GPU operator on the rows it received with its own ``local_expert_offset``
     (the receiver re-derives the routing from the logits, bit-identically), which yields one bf16
     row per (token, rank) already reduced over that rank's experts,
  4. returns those rows (second all-to-all) and sums each token's rows in rank order in fp32.
Experts that no participating rank owns (world size < 8) are dropped exactly as the single-GPU
operator drops non-local experts.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

EXPERTS_PER_RANK = 32


def plan_dispatch(topk_ids: torch.Tensor, world: int, experts_per_rank: int = EXPERTS_PER_RANK):
    """From the routing choices [T,8] derive the dispatch layout.

    Returns (send_tok int64 [S], send_counts int64 [world], pos int32 [T, world]): rows are sent in
    (destination rank, token) order; ``pos[t, g]`` is the row of token t in the block for rank g,
    counted over the whole send buffer, or -1.
    """
    T = topk_ids.shape[0]
    dest = topk_ids.long() // experts_per_rank                       # [T,8]
    mask = torch.zeros((T, max(world, int(256 // experts_per_rank))), dtype=torch.bool,
                       device=topk_ids.device)
    mask.scatter_(1, dest, torch.ones_like(dest, dtype=torch.bool))
    mask = mask[:, :world]
    gt = mask.t().contiguous().nonzero()                             # sorted by (rank, token)
    send_rank, send_tok = gt[:, 0], gt[:, 1]
    send_counts = mask.sum(dim=0).to(torch.int64)
    pos = torch.full((T, world), -1, dtype=torch.int32, device=topk_ids.device)
    pos[send_tok, send_rank] = torch.arange(send_tok.numel(), dtype=torch.int32, device=topk_ids.device)
    return send_tok, send_counts, pos


def pack_rows(hidden_states, hidden_states_scale, routing_logits, tok):
    """uint8 [S, H + 4*H/128 + 4*256]: e4m3 row | fp32 scales | fp32 logits of each sent token."""
    x = hidden_states.view(torch.uint8)[tok]
    sc = hidden_states_scale.t().contiguous()[tok].contiguous().view(torch.uint8).reshape(tok.numel(), -1)
    lg = routing_logits[tok].contiguous().view(torch.uint8).reshape(tok.numel(), -1)
    return torch.cat([x, sc, lg], dim=1).contiguous()


def unpack_rows(buf, hidden, fp8_dtype):
    R = buf.shape[0]
    nsc = hidden // 128
    x = buf[:, :hidden].contiguous().view(fp8_dtype)
    sc = buf[:, hidden:hidden + 4 * nsc].contiguous().view(torch.float32).reshape(R, nsc)
    lg = buf[:, hidden + 4 * nsc:].contiguous().view(torch.float32).reshape(R, 256)
    return x, sc.t().contiguous(), lg


def combine_rows_torch(rows_bf16, pos, out_dtype=torch.bfloat16):
    """Reference combine: fp32 sum in rank order (used on CPU and to check the CUDA kernel)."""
    T, G = pos.shape
    acc = torch.zeros((T, rows_bf16.shape[1]), dtype=torch.float32, device=rows_bf16.device)
    for g in range(G):
        p = pos[:, g].long()
        ok = p >= 0
        acc[ok] += rows_bf16[p[ok]].float()
    return acc.to(out_dtype)


class ExpertParallelMoE:
    """Expert-parallel wrapper; ``routing_fn`` / ``expert_fn`` / ``combine_fn`` default to the CUDA
    operators and can be replaced by CPU stand-ins to test the exchange logic under gloo."""

    kernels_per_step = 8  # routing + (routing, scatter, permute, 2 GEMMs, combine) + EP combine

    def __init__(self, rank: int, world: int, group=None, routing_fn=None, expert_fn=None,
                 combine_fn=None):
        self.rank, self.world, self.group = rank, world, group
        if routing_fn is None or expert_fn is None or combine_fn is None:
            from . import moe
            routing_fn = routing_fn or (lambda lg, b, f: moe.ds_routing(lg, b, f)[0])
            expert_fn = expert_fn or moe.run
            combine_fn = combine_fn or moe.ep_combine
        self.routing_fn, self.expert_fn, self.combine_fn = routing_fn, expert_fn, combine_fn
        self.backend = "nccl"

    def close(self):
        """Releases what the instance holds (nothing for the NCCL exchange)."""

    @torch.no_grad()
    def run(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
            gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor):
        T, H = hidden_states.shape
        dev = hidden_states.device
        ids = self.routing_fn(routing_logits, routing_bias, routed_scaling_factor)
        send_tok, send_counts, pos = plan_dispatch(ids, self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        # the split sizes of a variable all-to-all live on the host: one small device->host read
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        send_buf = pack_rows(hidden_states, hidden_states_scale, routing_logits, send_tok)
        recv_buf = torch.empty((sum(rc), send_buf.shape[1]), dtype=torch.uint8, device=dev)
        dist.all_to_all_single(recv_buf, send_buf, output_split_sizes=rc, input_split_sizes=sc,
                               group=self.group)
        x, xs, lg = unpack_rows(recv_buf, H, hidden_states.dtype)
        if x.shape[0] > 0:
            part = self.expert_fn(lg, routing_bias, x, xs, gemm1_weights, gemm1_weights_scale,
                                  gemm2_weights, gemm2_weights_scale,
                                  EXPERTS_PER_RANK * self.rank, routed_scaling_factor)
        else:
            part = torch.empty((0, H), dtype=torch.bfloat16, device=dev)
        back = torch.empty((sum(sc), H), dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(back, part.contiguous(), output_split_sizes=sc, input_split_sizes=rc,
                               group=self.group)
        return self.combine_fn(back, pos)
