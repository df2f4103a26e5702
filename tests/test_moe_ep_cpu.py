"""Expert-parallel exchange logic on CPU: world_size 2 over gloo with the CPU oracle standing in
for the CUDA operators (the host-side planning, packing, all-to-all and combine are the code under
test), plus single-process checks of the dispatch plan."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from ako4x_b200 import moe_ep, workloads as W

KEYS = ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
        "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale"]


def test_plan_dispatch_layout():
    ids = torch.tensor([[0, 1, 33, 40, 70, 200, 201, 255],      # ranks 0,1,2,6,7
                        [32, 33, 34, 35, 36, 37, 38, 39],       # rank 1 only
                        [64, 65, 66, 67, 68, 69, 70, 71]],      # rank 2 only
                       dtype=torch.int32)
    tok, counts, pos = moe_ep.plan_dispatch(ids, 2)
    assert counts.tolist() == [1, 2]
    assert tok.tolist() == [0, 0, 1]                # (rank0: t0), (rank1: t0, t1)
    assert pos.tolist() == [[0, 1], [-1, 2], [-1, -1]]
    tok8, counts8, pos8 = moe_ep.plan_dispatch(ids, 8)
    assert counts8.tolist() == [1, 2, 2, 0, 0, 0, 1, 1]
    assert int(counts8.sum()) == tok8.numel() == int((pos8 >= 0).sum())


def test_pack_unpack_roundtrip():
    a = W.make_moe(5, shape_id=3, num_local_experts=1, hidden=256, inter=128)
    tok = torch.tensor([4, 0, 0, 2])
    buf = moe_ep.pack_rows(a["hidden_states"], a["hidden_states_scale"], a["routing_logits"], tok)
    assert buf.shape == (4, 256 + 8 + 1024)
    x, xs, lg = moe_ep.unpack_rows(buf, 256, a["hidden_states"].dtype)
    assert torch.equal(x.view(torch.uint8), a["hidden_states"].view(torch.uint8)[tok])
    assert torch.equal(xs, a["hidden_states_scale"][:, tok])
    assert torch.equal(lg, a["routing_logits"][tok])


def _rank_inputs(rank, tokens):
    a = W.make_moe(tokens, shape_id=50 + rank, num_local_experts=32, hidden=256, inter=128,
                   local_expert_offset=32 * rank)
    # the router bias is a model parameter: identical on every rank
    a["routing_bias"] = 0.01 * torch.randn(256, generator=torch.Generator().manual_seed(7))
    return a


def _worker(rank, world, port, tokens, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        mine = _rank_inputs(rank, tokens[rank])
        ep = moe_ep.ExpertParallelMoE(
            rank, world,
            routing_fn=lambda lg, b, f: oracle.ds_routing(lg, b, f)[0],
            expert_fn=oracle.moe_fp8_block_scale,
            combine_fn=moe_ep.combine_rows_torch)
        out = ep.run(*[mine[k] for k in KEYS], mine["routed_scaling_factor"])
        # expected: every rank's experts applied to MY tokens, bf16 per rank, summed in rank order
        acc = torch.zeros(tokens[rank], 256, dtype=torch.float32)
        for g in range(world):
            wg = _rank_inputs(g, tokens[g])   # same seed and draw order as rank g's own weights
            part = oracle.moe_fp8_block_scale(
                mine["routing_logits"], mine["routing_bias"], mine["hidden_states"],
                mine["hidden_states_scale"], wg["gemm1_weights"], wg["gemm1_weights_scale"],
                wg["gemm2_weights"], wg["gemm2_weights_scale"], 32 * g, 2.5)
            acc += part.float()
        ref = acc.to(torch.bfloat16)
        # CPU matmuls sum in a batch-size dependent order, so a partial may flip one bf16 rounding
        err = (out.float() - ref.float()).abs()
        close = bool((err <= 1e-2 * ref.float().abs() + 1e-3).all())
        exact = (out == ref).float().mean().item()
        q.put((rank, close and exact > 0.98, bool((out != 0).any())))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_expert_parallel_equals_sum_over_ranks_world2():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    tokens = [24, 9]  # ragged: ranks hold different numbers of tokens
    procs = [ctx.Process(target=_worker, args=(r, world, port, tokens, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, equal, nonzero in res:
        assert equal, f"rank {rank}: expert-parallel result differs from the sum over ranks"
        assert nonzero, f"rank {rank}: no token reached a covered expert"
