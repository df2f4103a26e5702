"""The producers in front of the operator set and the indexer -> sparse attention chain, through the
C ABI: the FP8 activation quantiser and the index-K cache writer are compared bit for bit with their
CPU restatements; the chain must equal the two operators called one after the other."""
import pytest
import torch

import oracle
from ako4x_b200 import dsa_attention, dsa_indexer, fp8_quantize, moe, workloads as W
from conftest import assert_close_bf16, assert_lse_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 128), (3, 7168), (257, 7168), (64, 2048)])
def test_quantiser_bit_exact(built_lib, rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * torch.rand(rows, 1, generator=g) * 4).to(torch.bfloat16)
    x[0, :128] = 0                                   # an all-zero block: scale 1.0
    if rows > 2:
        x[2, 5] = 300.0                              # an outlier sets its block's scale
    q, s = fp8_quantize.quantize_1x128(x.cuda())
    rq, rs = oracle.fp8_quantize_1x128(x)
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
    # first-principles check of the rule itself: dequantised values within half an e4m3 step
    deq = q.cpu().float().reshape(rows, cols // 128, 128) * rs.t().unsqueeze(-1)
    err = (deq - x.float().reshape(rows, cols // 128, 128)).abs()
    assert (err <= rs.t().unsqueeze(-1) * 16.0 * 1.001 + 1e-30).all()   # 3 mantissa bits: step <= 32 at the top (ties land exactly on 16)


def test_quantiser_feeds_the_moe(built_lib):
    """bf16 activations -> quantiser -> MoE equals the MoE on the workload generator's own e4m3 pair
    (both follow the amax / 448 rule), so the producer's layout is the one the operator takes."""
    a = W.make_moe(64, shape_id=91, device="cuda", num_local_experts=4)
    a["routing_logits"][:, :4] += 4.0
    x_bf16 = (a["hidden_states"].float() *
              a["hidden_states_scale"].t().repeat_interleave(128, dim=1)).to(torch.bfloat16)
    q, s = fp8_quantize.quantize_1x128(x_bf16)
    keys = ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
            "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
            "routed_scaling_factor"]
    ref = moe.run(*[a[k] for k in keys])
    b = dict(a, hidden_states=q, hidden_states_scale=s)
    out = moe.run(*[b[k] for k in keys])
    rel = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
    assert rel < 2e-2   # requantising bf16-rounded activations moves a few e4m3 roundings


def test_index_k_cache_writer_bit_exact_and_readable(built_lib):
    g = torch.Generator().manual_seed(17)
    pages, tokens = 12, 300
    k = (torch.randn(tokens, 128, generator=g) * 3).to(torch.bfloat16)
    slots = torch.randperm(pages * 64, generator=g)[:tokens].to(torch.int32)
    slots[5] = -1
    cache = torch.zeros(pages, 8448, dtype=torch.uint8)
    ref = oracle.index_k_cache_write(k, slots, cache.clone())
    out = fp8_quantize.index_k_cache_write(k.cuda(), slots.cuda(), cache.cuda())
    assert torch.equal(out.cpu(), ref)
    # what the writer stored is what the indexer's oracle reads back
    vals, scales = oracle.unpack_index_cache(out.cpu())
    t = 7
    page, s = divmod(int(slots[t]), 64)
    deq = vals[page, s] * scales[page, s]
    assert (deq - k[t].float()).abs().max() <= scales[page, s] * 16.0 * 1.001


@pytest.mark.parametrize("tokens,ctx", [(3, 1500), (24, 6000)])
def test_indexer_attention_chain(built_lib, tokens, ctx):
    a = W.make_dsa_indexer(tokens, ctx, shape_id=93, device="cuda")
    ikeys = ["q_index_fp8", "k_index_cache_fp8", "weights", "seq_lens", "block_table"]
    (idx,) = dsa_indexer.run(*[a[k] for k in ikeys])
    npages = a["k_index_cache_fp8"].shape[0]
    b = W.make_dsa_attention(tokens, ctx, idx, npages, shape_id=94, device="cuda")
    o, lse = dsa_attention.run(b["q_nope"], b["q_pe"], b["ckv_cache"], b["kpe_cache"], idx, b["sm_scale"])
    o2, lse2, idx2 = dsa_indexer.run_with_attention(*[a[k] for k in ikeys], b["q_nope"], b["q_pe"], b["ckv_cache"],
                                                    b["kpe_cache"], b["sm_scale"])
    assert torch.equal(idx2, idx)
    assert torch.equal(o2, o) and torch.equal(lse2, lse)
    c = {k: v.cpu() if torch.is_tensor(v) else v for k, v in b.items()}
    ro, rlse = oracle.dsa_sparse_attention(c["q_nope"], c["q_pe"], c["ckv_cache"], c["kpe_cache"], idx.cpu(),
                                           c["sm_scale"])
    assert_close_bf16(o2, ro)
    assert_lse_close(lse2, rlse)
