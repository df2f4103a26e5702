"""Generates the golden fixtures in this directory.

The operator definitions the reference is scored against (FlashInfer-Bench ``definition.json``
reference functions) are not vendored in the reference repository; flashinfer-python 0.6.11 ships
them as ``flashinfer.trace.templates``. This script imports those functions (they run on CPU),
feeds them small seeded inputs and stores inputs + outputs. It needs flashinfer-python and is run
by hand; the tests only read the ``.pt`` files it wrote.

    python tests/golden/make_golden.py

No definition exists for the DSA top-k indexer, so its fixture is produced by ``oracle.indexer``
itself (a regression guard, not a pin).
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from ako4x_b200 import workloads as W  # noqa: E402
import oracle  # noqa: E402

OUT = Path(__file__).resolve().parent


def _save(name, inputs, outputs):
    torch.save({"inputs": inputs, "outputs": outputs}, OUT / f"{name}.pt")
    size = (OUT / f"{name}.pt").stat().st_size
    print(f"{name}.pt  {size / 1024:.1f} KiB")


def main():
    from flashinfer.trace.templates import attention as A
    from flashinfer.trace.templates import moe as M
    from flashinfer.trace.templates import norm as N

    # RMSNorm: rows 1, 7, 64
    for i, rows in enumerate((1, 7, 64)):
        a = W.make_rmsnorm(rows, shape_id=900 + i)
        _save(f"rmsnorm_r{rows}", a, {"output": N._rmsnorm_reference(a["hidden_states"], a["weight"])})

    # GQA decode: ragged lengths with an empty sequence
    a = W.make_gqa_decode(4, shape_id=900, lens=[5, 0, 33, 17], extra_pages=7)
    o, lse = A._gqa_paged_decode_reference(a["q"], a["k_cache"], a["v_cache"], a["kv_indptr"],
                                           a["kv_indices"], a["sm_scale"])
    _save("gqa_decode_b4", a, {"output": o, "lse": lse})

    # MLA decode
    a = W.make_mla_decode(3, shape_id=900, lens=[9, 0, 70], extra_pages=5)
    o, lse = A._mla_paged_decode_reference(a["q_nope"], a["q_pe"], a["ckv_cache"], a["kpe_cache"],
                                           a["kv_indptr"], a["kv_indices"], a["sm_scale"])
    _save("mla_decode_b3", a, {"output": o, "lse": lse})

    # MLA prefill: includes q_len == kv_len and a sequence with a long prefix
    a = W.make_mla_prefill(3, shape_id=900, q_lens=[4, 6, 1], kv_lens=[4, 19, 8], extra_pages=5)
    o, lse = A._mla_paged_prefill_reference(a["q_nope"], a["q_pe"], a["ckv_cache"], a["kpe_cache"],
                                            a["qo_indptr"], a["kv_indptr"], a["kv_indices"],
                                            a["sm_scale"])
    _save("mla_prefill_b3", a, {"output": o, "lse": lse})

    # DSA sparse attention: rows with -1 holes, an all -1 row
    g = torch.Generator().manual_seed(W.BASE_SEED + 5900)
    pages = 3
    idx = torch.full((4, 48), -1, dtype=torch.int32)
    idx[0, :48] = torch.randperm(pages * 64, generator=g)[:48].to(torch.int32)
    idx[1, :20] = torch.randperm(pages * 64, generator=g)[:20].to(torch.int32)
    idx[2, 5:30:2] = torch.randperm(pages * 64, generator=g)[:13].to(torch.int32)
    a = W.make_dsa_attention(4, pages * 64, idx, pages, shape_id=900)
    o, lse = A._dsa_paged_reference(a["q_nope"], a["q_pe"], a["ckv_cache"], a["kpe_cache"],
                                    a["sparse_indices"], a["sm_scale"])
    _save("dsa_attention_t4", a, {"output": o, "lse": lse})

    # MoE at reduced hidden/intermediate sizes (routing is full size: 256 experts, 8 groups)
    a = W.make_moe(24, shape_id=900, num_local_experts=8, hidden=256, inter=128,
                   local_expert_offset=64)
    out = M._trtllm_fp8_block_scale_moe_ds_routing_reference(
        a["routing_logits"], a["routing_bias"], a["hidden_states"], a["hidden_states_scale"],
        a["gemm1_weights"], a["gemm1_weights_scale"], a["gemm2_weights"], a["gemm2_weights_scale"],
        8, 8, 4, a["local_expert_offset"], a["routed_scaling_factor"])
    _save("moe_t24_e8_h256_i128", a, {"output": out})

    # DSA indexer: oracle-generated (unpinned)
    a = W.make_dsa_indexer(3, 2048 + 130, shape_id=900, extra_pages=2)
    (topk,) = oracle.dsa_topk_indexer(a["q_index_fp8"], a["k_index_cache_fp8"], a["weights"],
                                      a["seq_lens"], a["block_table"])
    _save("dsa_indexer_t3", a, {"topk_indices": topk})


if __name__ == "__main__":
    main()
