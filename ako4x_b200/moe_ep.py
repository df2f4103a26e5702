"""Expert-parallel FP8 MoE: one process per GPU, rank r owns experts [32r, 32r+32) (with 8 groups
of 32 experts that is exactly routing group r, so a token reaches at most 4 ranks).

The reference has no distributed path; this module is the multi-GPU form of the operator in
``moe.py``. Two exchanges are implemented behind one class:

``backend="p2p"`` (the default on GPUs): every rank owns one buffer of peer-addressable memory
(torch symmetric memory: the same allocation mapped into every process of the group). One C-ABI
call per step (``ako4x_moe_fp8_block_scale_ep``) routes the rank's tokens, STORES each token row
(e4m3 row, 56 scales, 8 expert ids, 8 weights) straight into the receive area of every rank that owns
one of its experts, runs the operator on the rows it received, stores every row's bf16 partial back
into the sender's return area, and sums each token's partials in rank order. Kernels signal each
other through step counters in the peers' memory; there is no collective call and no host
synchronisation in a step.

``backend="nccl"``: the same exchange with ``all_to_all_single`` (three collectives and one host
read of the split sizes per step); it also runs on CPU under gloo with stand-in operators, which is
how the host-side logic is tested without GPUs. Per step every rank
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

    def __init__(self, rank: int, world: int, group=None, routing_fn=None, expert_fn=None,
                 combine_fn=None, backend=None):
        self.rank, self.world, self.group = rank, world, group
        custom = routing_fn is not None or expert_fn is not None or combine_fn is not None
        if backend is None:
            backend = "nccl" if custom or not torch.cuda.is_available() else "p2p"
        if backend not in ("p2p", "nccl"):
            raise ValueError("backend must be 'p2p' or 'nccl'")
        self.backend = backend
        if backend == "nccl" and (routing_fn is None or expert_fn is None or combine_fn is None):
            from . import moe
            routing_fn = routing_fn or (lambda lg, b, f: moe.ds_routing(lg, b, f)[0])
            expert_fn = expert_fn or moe.run
            combine_fn = combine_fn or moe.ep_combine
        self.routing_fn, self.expert_fn, self.combine_fn = routing_fn, expert_fn, combine_fn
        # p2p state: the peer-addressable buffer, the private workspace, the step counter
        self._cap = 0
        self._buf = self._hdl = self._ws = self._peers = None
        self._step = 0

    @property
    def kernels_per_step(self) -> int:
        # p2p: routing, plan, send | recv-route, scatter, permute, GEMM1, GEMM2, return | finish
        # nccl: routing + (routing, scatter, permute, 2 GEMMs, combine) + EP combine
        return 10 if self.backend == "p2p" else 8

    def close(self):
        """Releases the peer-addressable buffer and the workspace (after a barrier: no peer may
        still be storing into them)."""
        if self._buf is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self._buf = self._hdl = self._ws = self._peers = None
            self._cap = 0

    def status(self) -> int:
        """0, or the code of a bounded wait on a peer that gave up (synchronises the device)."""
        if self._buf is None:
            return 0
        from . import _cabi
        return int(_cabi.lib().ako4x_moe_ep_status(self._buf.data_ptr()))

    def _ensure_p2p(self, tokens: int, device) -> None:
        """(Re)allocates the buffers when a step brings more tokens than any before. Collective:
        every rank must call it with the same step count (the capacity is the maximum over ranks)."""
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        from . import _cabi
        t = torch.tensor([tokens], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        cap = max(int(t.item()), 1)
        if cap <= self._cap:
            return
        self.close()
        L = _cabi.lib()
        grp = self.group if self.group is not None else dist.group.WORLD
        nbytes = L.ako4x_moe_ep_buffer_bytes(self.world, cap)
        self._buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self._hdl = symm_mem.rendezvous(self._buf, grp.group_name)
        self._buf[:4096].zero_()                  # the flag block: step counters start at 0
        torch.cuda.synchronize()
        dist.barrier(group=self.group)            # nobody stores into a buffer that is not zeroed yet
        ptrs = [int(x) for x in self._hdl.buffer_ptrs]
        self._peers = (ctypes.c_void_p * self.world)(*ptrs)
        self._cap = cap
        self._pairs = 2 * self.world * cap        # twice the (token, expert) pairs of uniform routing
        ws_bytes = L.ako4x_moe_ep_workspace_bytes(cap, self.world, cap, self._pairs)
        self._ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        self._step = 0

    @torch.no_grad()
    def _run_p2p(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                 gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor):
        from . import _cabi
        T, H = hidden_states.shape
        dev = hidden_states.device
        if gemm1_weights.shape[0] != EXPERTS_PER_RANK:
            raise _cabi.Ako4xError("moe_ep: every rank holds 32 experts")
        if T > self._cap:
            raise _cabi.Ako4xError("moe_ep: call prepare(tokens) on every rank before a larger step")
        out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        keep = [t.contiguous() for t in (routing_logits, routing_bias, hidden_states, hidden_states_scale,
                                         gemm1_weights_scale, gemm2_weights_scale)]
        self._step += 1
        st = _cabi.lib().ako4x_moe_fp8_block_scale_ep(
            _cabi.ptr(keep[0]), _cabi.ptr(keep[1]), 1 if routing_bias.dtype == torch.bfloat16 else 0,
            _cabi.ptr(keep[2]), _cabi.ptr(keep[3]), _cabi.ptr(gemm1_weights), _cabi.ptr(keep[4]),
            _cabi.ptr(gemm2_weights), _cabi.ptr(keep[5]), float(routed_scaling_factor), _cabi.ptr(out), T,
            self.world, self.rank, self._cap, self._pairs, self._step, self._peers, _cabi.ptr(self._ws),
            self._ws.numel(), _cabi.stream())
        del keep
        _cabi.check(st, "ako4x_moe_fp8_block_scale_ep")
        return out

    def prepare(self, tokens: int, device=None) -> None:
        """Collective set-up for steps of up to `tokens` tokens per rank (p2p backend): allocates and
        maps the exchange buffers. ``run`` calls it on first use; call it explicitly before a step
        that is larger than any earlier one, and before capturing steps in a CUDA graph."""
        if self.backend == "p2p":
            self._ensure_p2p(tokens, device or torch.device("cuda", torch.cuda.current_device()))

    @torch.no_grad()
    def run(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
            gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor):
        T, H = hidden_states.shape
        dev = hidden_states.device
        if self.backend == "p2p":
            if self._buf is None:
                self._ensure_p2p(T, dev)
            return self._run_p2p(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                                 gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, routed_scaling_factor)
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
