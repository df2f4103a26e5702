"""The CPU oracle against the golden fixtures (outputs of the FlashInfer-Bench operator
definitions on small seeded inputs, see tests/golden/make_golden.py). Runs without a GPU."""
import pytest
import torch

import oracle
from conftest import GOLDEN, assert_close_bf16, assert_lse_close, load_golden


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


def _bf16_ordinal(x: torch.Tensor) -> torch.Tensor:
    """Monotone integer image of the bf16 rounding of fp32 values (adjacent bf16 values differ by 1)."""
    bits = x.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    return torch.where(bits >= 0x8000, 0x8000 - bits, bits)   # negative values below positive ones


def test_indexer_oracle_against_the_reference_kernel_outputs():
    """Pins oracle/indexer.py to outputs of the reference's own GPU kernel
    (reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py::run), recorded on a B200 by
    tests/golden/make_indexer_reference_golden.py on inputs this test redraws from the same seeds.

    The reference ranks bf16-rounded scores and emits an unordered set, so the comparison is per
    row and by set: rows of at most 2048 tokens must be identical (the listing rule, order
    included); for longer rows every slot that only one side selected must have an oracle score
    whose bf16 rounding is the bf16 rounding of the 2048-th best score, give or take one bf16 step
    (the reference's fp32 sums run in another order before they are rounded)."""
    import hashlib
    from ako4x_b200 import workloads as W
    g = torch.load(GOLDEN / "dsa_indexer_reference_v8.pt", weights_only=True)
    keys = ["q_index_fp8", "k_index_cache_fp8", "weights", "seq_lens", "block_table"]
    checked_long_rows = 0
    for case in g["cases"]:
        a = W.make_dsa_indexer(case["rows"], case["ctx"], shape_id=case["shape_id"], device="cpu")
        h = hashlib.sha256()
        for k in keys:
            h.update(a[k].contiguous().view(torch.uint8).numpy().tobytes())
        assert h.hexdigest() == case["input_sha256"], "the seeded inputs are not the recorded ones"
        scores = oracle.dsa_index_scores(*[a[k] for k in keys])
        mine = oracle.dsa_topk_select(scores, a["seq_lens"], a["block_table"])
        ref = case["topk_indices"]
        assert ref.shape == mine.shape
        # global slot -> token position of this sequence (one block table for all rows)
        bt = a["block_table"][0].long()
        pos_of_slot = {int(bt[p]) * 64 + s: p * 64 + s for p in range(bt.numel()) for s in range(64)}
        for r in range(case["rows"]):
            sl = int(a["seq_lens"][r])
            if sl <= 2048:
                assert torch.equal(ref[r], mine[r]), f"ctx {case['ctx']} row {r}: listing differs"
                continue
            checked_long_rows += 1
            rs, ms = set(ref[r].tolist()), set(mine[r].tolist())
            assert -1 not in rs and len(rs) == 2048 and len(ms) == 2048
            diff = rs ^ ms
            row = scores[r, :sl]
            kth = torch.sort(row, descending=True).values[2047]
            kth_ord = int(_bf16_ordinal(kth.reshape(1)))
            for slot in diff:
                o = int(_bf16_ordinal(row[pos_of_slot[slot]].reshape(1)))
                assert abs(o - kth_ord) <= 1, (f"ctx {case['ctx']} row {r}: slot {slot} differs from the "
                                               f"reference and is not a bf16 tie of the 2048-th score")
            assert len(diff) <= 2 * 64, f"ctx {case['ctx']} row {r}: {len(diff)} slots differ"
    assert checked_long_rows >= 9


@pytest.mark.parametrize("name", ["gdn_decode_b2", "gdn_decode_b1_nostate"])
def test_gdn_decode(name):
    """oracle.gdn_decode against the FlashInfer-Bench definition's outputs. fp32 sums in another
    order: state within 2e-6 relative to the row scale, bf16 output within one rounding step."""
    from ako4x_b200 import workloads as W
    g = load_golden(name)
    i = g["inputs"]
    a = W.make_gdn_decode(i["batch"], shape_id=i["shape_id"], with_state=i["with_state"])
    for key in ("q", "k", "v", "A_log", "a", "dt_bias", "b"):
        assert torch.equal(a[key], i[key]), key
    if i["with_state"]:
        assert a["state"].double().sum().item() == i["state_digest"]
    o, s = oracle.gdn_decode(a["q"], a["k"], a["v"], a["state"], a["A_log"], a["a"], a["dt_bias"], a["b"], a["scale"])
    ref_o, ref_s = g["outputs"]["output"], g["outputs"]["new_state"]
    assert o.shape == ref_o.shape and o.dtype == torch.bfloat16 and s.shape == ref_s.shape
    assert (s - ref_s).abs().max().item() <= 2e-6 * ref_s.abs().max().item() + 1e-7
    assert_close_bf16(o, ref_o, atol=1e-4, rtol=1e-2)
    assert (o == ref_o).float().mean().item() > 0.97


@pytest.mark.parametrize("m", [1, 37, 200])
def test_gemm(m):
    """oracle.gemm_nt against torch.matmul(A, B.T) on fp16 tensors (the reference expression of the
    family): fp32 sums in another order, so a value may round to the neighbouring fp16."""
    from ako4x_b200 import workloads as W
    g = load_golden(f"gemm_m{m}")
    a = W.make_gemm(m, shape_id=g["inputs"]["shape_id"])
    assert (a["A"].double().sum() + a["B"].double().sum()).item() == g["inputs"]["digest"]
    c = oracle.gemm_nt(a["A"], a["B"])
    ref = g["outputs"]["C"]
    assert c.shape == ref.shape and c.dtype == torch.float16
    err = (c.float() - ref.float()).abs()
    assert (err <= 2e-3 * ref.float().abs() + 1e-2).all()
    assert (c == ref).float().mean().item() > 0.97


def test_gdn_prefill():
    """oracle.gdn_prefill against the FlashInfer-Bench definition (three packed sequences, one
    empty)."""
    from ako4x_b200 import workloads as W
    g = load_golden("gdn_prefill_s3")
    a = W.make_gdn_prefill(g["inputs"]["seq_lens"], shape_id=g["inputs"]["shape_id"])
    assert a["state"].double().sum().item() == g["inputs"]["state_digest"]
    o, s = oracle.gdn_prefill(a["q"], a["k"], a["v"], a["state"], a["A_log"], a["a"], a["dt_bias"], a["b"],
                              a["cu_seqlens"], a["scale"])
    ref_o, ref_s = g["outputs"]["output"], g["outputs"]["new_state"]
    assert (s - ref_s).abs().max().item() <= 1e-5 * ref_s.abs().max().item()
    assert torch.all(ref_s[1] == 0) and torch.all(s[1] == 0)
    assert_close_bf16(o, ref_o, atol=1e-3, rtol=1e-2)
    assert (o == ref_o).float().mean().item() > 0.95
