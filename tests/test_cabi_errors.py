"""Argument validation of the C ABI: bad calls return a status and launch nothing, so these run
without a GPU (every call below is rejected, or is a zero-size no-op, before any CUDA call)."""
import ctypes

import pytest

from ako4x_b200 import _cabi

OK, EINVAL, EWORKSPACE = 0, -1, -4
P = ctypes.c_void_p


@pytest.fixture(scope="module")
def L(built_lib):
    return _cabi.lib()


def _buf(nbytes=4096, offset=0):
    """A host buffer standing in for a device pointer: validation never dereferences it."""
    raw = ctypes.create_string_buffer(nbytes + 512)
    base = (ctypes.addressof(raw) + 255) & ~255
    return raw, base + offset


def test_abi_version(L):
    assert L.ako4x_abi_version() >= 1


def test_rmsnorm_validation(L):
    keep, x = _buf()
    assert L.ako4x_rmsnorm_h128(None, x, x, 4, None) == EINVAL
    assert L.ako4x_rmsnorm_h128(x, x, x, -1, None) == EINVAL
    assert L.ako4x_rmsnorm_h128(x, x, x, 0, None) == OK          # nothing to do


def test_gqa_validation(L):
    keep, x = _buf()
    f = L.ako4x_gqa_paged_decode
    assert f(None, x, x, x, x, 0.1, x, x, 1, 8, 1, None, 0, None) == EINVAL
    assert f(x, x, x, x, x, 0.1, x, x, -1, 8, 1, None, 0, None) == EINVAL
    assert f(x, x, x, x, x, 0.1, x, x, 0, 0, 1, None, 0, None) == OK
    # a batch that needs split-KV partials without a workspace
    need = L.ako4x_gqa_paged_decode_workspace_bytes(1, 8192, 1)
    assert need > 0
    assert f(x, x, x, x, x, 0.1, x, x, 1, 8192, 1, None, 0, None) == EWORKSPACE


def test_mla_decode_and_prefill_validation(L):
    keep, x = _buf()
    keep2, odd = _buf(offset=8)                                  # 8-byte aligned only
    d = L.ako4x_mla_paged_decode
    assert d(None, x, x, x, x, x, 0.1, x, x, 1, 8, 1, None, 0, None) == EINVAL
    assert d(odd, x, x, x, x, x, 0.1, x, x, 1, 8, 1, None, 0, None) == EINVAL      # misaligned q_nope
    assert d(x, x, x, x, x, x, 0.1, x, x, 0, 0, 1, None, 0, None) == OK
    pf = L.ako4x_mla_paged_prefill
    assert pf(x, x, x, x, None, x, x, 0.1, x, x, 64, 1, 64, 1, None, 0, None) == EINVAL
    assert pf(x, x, x, x, x, x, x, 0.1, x, x, 64, 0, 64, 1, None, 0, None) == EINVAL   # rows but no sequences
    assert pf(x, x, x, x, x, x, x, 0.1, x, x, 0, 1, 0, 1, None, 0, None) == OK
    # 64 query tokens take the tensor-core path, which needs its key copies
    need = L.ako4x_mla_paged_prefill_workspace_bytes(64, 1, 64, 1)
    assert need >= 64 * 2176
    assert L.ako4x_mla_paged_prefill_workspace_bytes(8, 1, 64, 1) == 0
    assert pf(x, x, x, x, x, x, x, 0.1, x, x, 64, 1, 64, 1, None, 0, None) == EWORKSPACE


def test_indexer_validation(L):
    keep, x = _buf()
    f = L.ako4x_dsa_topk_indexer
    assert f(None, x, x, x, x, x, 1, 64, 80, None, 0, None) == EINVAL
    assert f(x, x, x, x, x, x, -1, 64, 80, None, 0, None) == EINVAL
    assert f(x, x, x, x, x, x, 0, 64, 80, None, 0, None) == OK
    assert L.ako4x_dsa_topk_indexer_workspace_bytes(2, 64) == 2 * 64 * 64 * 4
    assert f(x, x, x, x, x, x, 2, 64, 80, None, 0, None) == EWORKSPACE
    assert L.ako4x_dsa_topk_select(None, x, x, x, 1, 64, None) == EINVAL


def test_sparse_attention_and_moe_validation(L):
    keep, x = _buf()
    sa = L.ako4x_dsa_sparse_attention
    assert sa(None, x, x, x, x, 0.1, x, x, 1, 2048, 100, None, 0, None) == EINVAL
    assert sa(x, x, x, x, x, 0.1, x, x, 0, 2048, 100, None, 0, None) == OK
    moe = L.ako4x_moe_fp8_block_scale
    assert moe(None, x, 0, x, x, x, x, x, x, 0, 2.5, x, 8, 32, None, 0, None) == EINVAL
    need = L.ako4x_moe_fp8_block_scale_workspace_bytes(8, 32)
    assert need > 0
    assert moe(x, x, 0, x, x, x, x, x, x, 0, 2.5, x, 8, 32, None, 0, None) == EWORKSPACE
