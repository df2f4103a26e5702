"""The shared library loads and exports every function the public header declares (no compute)."""
import ctypes

from ako4x_b200 import _cabi


def test_header_declares_expected_entry_points():
    names = _cabi.declared_symbols()
    for must in ("ako4x_rmsnorm_h128", "ako4x_gqa_paged_decode", "ako4x_mla_paged_decode",
                 "ako4x_mla_paged_prefill", "ako4x_dsa_topk_indexer", "ako4x_dsa_sparse_attention",
                 "ako4x_moe_fp8_block_scale"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    missing = [n for n in _cabi.declared_symbols() if not hasattr(built_lib, n)]
    assert not missing, f"declared in include/ako4x_b200.h but not exported: {missing}"


def test_every_declared_symbol_has_a_ctypes_signature():
    missing = [n for n in _cabi.declared_symbols() if n not in _cabi._SIGNATURES]
    assert not missing


def test_abi_version(built_lib):
    assert built_lib.ako4x_abi_version() >= 1


def test_argument_validation_without_gpu(built_lib):
    """Status codes that are decided before any CUDA call."""
    assert built_lib.ako4x_rmsnorm_h128(None, None, None, -1, None) == -1
    assert built_lib.ako4x_rmsnorm_h128(None, None, None, 0, None) == 0
    assert built_lib.ako4x_rmsnorm_h128(None, None, None, 4, None) == -1
    assert built_lib.ako4x_gqa_paged_decode(None, None, None, None, None, 1.0, None, None, 0, 0, 1,
                                            None, 0, None) == 0
    assert built_lib.ako4x_gqa_paged_decode(None, None, None, None, None, 1.0, None, None, 2, 0, 0,
                                            None, 0, None) == -1
    assert built_lib.ako4x_gqa_paged_decode_workspace_bytes(256, 256 * 4096, 1) > 0
    assert built_lib.ako4x_dsa_topk_indexer_workspace_bytes(2, 10) == 2 * 10 * 64 * 4


def test_missing_library_raises(monkeypatch, tmp_path):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "nope.so")
    try:
        _cabi.lib()
    except _cabi.Ako4xError as e:
        assert "no fallback" in str(e)
    else:
        raise AssertionError("a missing library must raise")


def test_cpu_tensors_are_rejected(built_lib):
    import torch
    from ako4x_b200 import rmsnorm
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    w = torch.ones(128, dtype=torch.bfloat16)
    try:
        rmsnorm.run(x, w)
    except _cabi.Ako4xError as e:
        assert "CUDA" in str(e)
    else:
        raise AssertionError("CPU tensors must be rejected: there is no CPU path")
