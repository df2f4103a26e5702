"""The packed-solution folders: the layout the reference's packer requires
(scripts/pack_solution.py:38-106 of the reference) and entry points with the reference's exact
parameter lists. Runs without a GPU (nothing is launched)."""
import importlib.util
import inspect
import tomllib
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
SOLUTIONS = sorted(p for p in (ROOT / "solutions").iterdir() if p.is_dir())

PARAMS = {
    "rmsnorm_h128": ["hidden_states", "weight"],
    "gqa_paged_decode_h32_kv8_d128_ps1": ["q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "sm_scale"],
    "mla_paged_decode_h16_ckv512_kpe64_ps1": ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "kv_indptr", "kv_indices",
                                              "sm_scale"],
    "mla_paged_prefill_causal_h16_ckv512_kpe64_ps1": ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "qo_indptr",
                                                      "kv_indptr", "kv_indices", "sm_scale"],
    "dsa_topk_indexer_fp8_h64_d128_topk2048_ps64": ["q_index_fp8", "k_index_cache_fp8", "weights", "seq_lens",
                                                    "block_table"],
    "dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64": ["q_nope", "q_pe", "ckv_cache", "kpe_cache",
                                                            "sparse_indices", "sm_scale"],
    "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048": [
        "routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
        "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
        "routed_scaling_factor"],
    "gemm_n2048_k4096": ["A", "B"],
    "gdn_prefill_qk4_v8_d128_k_last": ["q", "k", "v", "state", "A_log", "a", "dt_bias", "b", "cu_seqlens", "scale"],
    "gdn_decode_qk4_v8_d128_k_last": ["q", "k", "v", "state", "A_log", "a", "dt_bias", "b", "scale"],
}


def test_every_operator_has_a_solution_folder():
    assert sorted(p.name for p in SOLUTIONS) == sorted(PARAMS)


@pytest.mark.parametrize("folder", SOLUTIONS, ids=lambda p: p.name)
def test_config_has_what_the_packer_requires(folder):
    cfg = tomllib.loads((folder / "config.toml").read_text())
    for key in ("name", "definition", "author"):
        assert key in cfg["solution"]
    for key in ("language", "entry_point"):
        assert key in cfg["build"]
    assert cfg["solution"]["definition"] == folder.name
    assert cfg["build"]["language"] == "python"
    assert cfg["build"]["entry_point"] == "kernel.py::run"
    assert cfg["build"].get("destination_passing_style", False) is False
    assert (folder / "solution" / "kernel.py").exists()


@pytest.mark.parametrize("folder", SOLUTIONS, ids=lambda p: p.name)
def test_entry_point_keeps_the_reference_parameter_list(folder):
    spec = importlib.util.spec_from_file_location(f"solution_{folder.name}", folder / "solution" / "kernel.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    params = [p for p in inspect.signature(mod.run).parameters if not p.startswith("_")]
    assert params == PARAMS[folder.name]
