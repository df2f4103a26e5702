"""The CPU oracle against the golden fixtures (outputs of the FlashInfer-Bench operator
definitions on small seeded inputs, see tests/golden/make_golden.py). Runs without a GPU."""
import pytest
import torch

import oracle
from conftest import assert_close_bf16, assert_lse_close, load_golden


@pytest.mark.parametrize("rows", [1, 7, 64])
def test_rmsnorm(rows):
    g = load_golden(f"rmsnorm_r{rows}")
    out = oracle.rmsnorm(g["inputs"]["hidden_states"], g["inputs"]["weight"])
    assert torch.equal(out, g["outputs"]["output"])  # same fp32 arithmetic: bit-exact


def _attn(name, fn, keys):
    g = load_golden(name)
    i = g["inputs"]
    o, lse = fn(*[i[k] for k in keys])
    # bf16 outputs may differ by one rounding step where fp32 sums are ordered differently
    assert_close_bf16(o, g["outputs"]["output"], atol=1e-2, rtol=1e-2)
    assert_lse_close(lse, g["outputs"]["lse"], tol=1e-5)
    frac_exact = (o == g["outputs"]["output"]).float().mean().item()
    assert frac_exact > 0.98


def test_gqa_decode():
    _attn("gqa_decode_b4", oracle.gqa_paged_decode,
          ["q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "sm_scale"])


def test_mla_decode():
    _attn("mla_decode_b3", oracle.mla_paged_decode,
          ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "kv_indptr", "kv_indices", "sm_scale"])


def test_mla_prefill():
    _attn("mla_prefill_b3", oracle.mla_paged_prefill,
          ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "qo_indptr", "kv_indptr", "kv_indices",
           "sm_scale"])


def test_dsa_sparse_attention():
    _attn("dsa_attention_t4", oracle.dsa_sparse_attention,
          ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "sparse_indices", "sm_scale"])
    g = load_golden("dsa_attention_t4")
    # the all -1 row: zero output, -inf lse
    assert torch.all(g["outputs"]["output"][3] == 0) and torch.isinf(g["outputs"]["lse"][3]).all()


def test_moe():
    g = load_golden("moe_t24_e8_h256_i128")
    i = g["inputs"]
    out = oracle.moe_fp8_block_scale(
        i["routing_logits"], i["routing_bias"], i["hidden_states"], i["hidden_states_scale"],
        i["gemm1_weights"], i["gemm1_weights_scale"], i["gemm2_weights"], i["gemm2_weights_scale"],
        i["local_expert_offset"], i["routed_scaling_factor"])
    ref = g["outputs"]["output"]
    assert (ref != 0).any(), "fixture routes no token to a local expert"
    assert_close_bf16(out, ref, atol=1e-2, rtol=1e-2)


def test_moe_routing_matches_topk_definition():
    """Expert sets of the stable-sort routing equal torch.topk's on tie-free inputs."""
    g = load_golden("moe_t24_e8_h256_i128")
    i = g["inputs"]
    ids, w = oracle.ds_routing(i["routing_logits"], i["routing_bias"], i["routed_scaling_factor"])
    s = torch.sigmoid(i["routing_logits"].float())
    sb = s + i["routing_bias"].float()
    gs = sb.view(-1, 8, 32).topk(2, dim=2).values.sum(2)
    keep = torch.zeros_like(gs).scatter_(1, gs.topk(4, dim=1).indices, 1.0)
    pruned = sb.masked_fill(keep.repeat_interleave(32, dim=1) == 0, float("-inf"))
    ref_ids = pruned.topk(8, dim=1).indices.sort(dim=1).values
    assert torch.equal(ids.long(), ref_ids)
    assert torch.allclose(w.sum(1), torch.full((ids.shape[0],), 2.5), atol=1e-5)


def test_indexer_regression_fixture():
    g = load_golden("dsa_indexer_t3")
    i = g["inputs"]
    (topk,) = oracle.dsa_topk_indexer(i["q_index_fp8"], i["k_index_cache_fp8"], i["weights"],
                                      i["seq_lens"], i["block_table"])
    assert torch.equal(topk, g["outputs"]["topk_indices"])


def test_indexer_selection_rules():
    """Ties go to the lower position; short rows list every token; output is in position order."""
    bt = torch.tensor([[3, 1, 0, 2] + list(range(4, 40))], dtype=torch.int32)
    sl = torch.tensor([2100], dtype=torch.int32)
    scores = torch.zeros(1, 40 * 64)
    scores[0, 10] = 5.0
    scores[0, 2099] = 7.0
    out = oracle.dsa_topk_select(scores, sl, bt)
    pos = [0] * 0
    # 2 distinct winners + the first 2046 zeros by position
    exp_pos = sorted({10, 2099} | set([p for p in range(2100) if p not in (10, 2099)][:2046]))
    exp = torch.tensor([int(bt[0, p // 64]) * 64 + p % 64 for p in exp_pos], dtype=torch.int32)
    assert torch.equal(out[0], exp)
    out = oracle.dsa_topk_select(scores, torch.tensor([70], dtype=torch.int32), bt)
    assert out[0, :70].tolist() == [int(bt[0, p // 64]) * 64 + p % 64 for p in range(70)]
    assert (out[0, 70:] == -1).all()
