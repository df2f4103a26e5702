"""The scratch-free GQA decode entry point (ako4x_gqa_paged_decode_noalloc) against the regular
one, called through the C ABI.

This entry point exists for callers that can pass inputs and outputs but no workspace, and that
may not allocate device memory themselves: a plug-in host with a fixed (inputs, outputs) calling
convention, or a server whose HBM is already fully handed to its KV-cache pool. Its split-KV
partials live in one array inside the library, shared by all calls on the device, so the test
makes two calls in a row with different inputs: the second call sees the first call's leftovers
in the array and must still agree with the regular entry point.

The file name sorts last on purpose, so that a run which stops at the first failure has already
run every other test.
"""
import pytest
import torch

import oracle
from ako4x_b200 import _cabi, gqa_decode, workloads as W
from conftest import assert_close_bf16, assert_lse_close

pytestmark = pytest.mark.gpu
KEYS = ["q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "sm_scale"]


def _noalloc(a):
    """Calls the C entry point directly: outputs come from the caller, nothing else is passed."""
    L = _cabi.lib()
    batch = a["q"].shape[0]
    o = torch.full_like(a["q"], float("nan"))
    lse = torch.full((batch, 32), float("nan"), dtype=torch.float32, device=a["q"].device)
    st = L.ako4x_gqa_paged_decode_noalloc(
        a["q"].data_ptr(), a["k_cache"].data_ptr(), a["v_cache"].data_ptr(),
        a["kv_indptr"].data_ptr(), a["kv_indices"].data_ptr(), float(a["sm_scale"]),
        o.data_ptr(), lse.data_ptr(), batch, a["kv_indices"].numel(), a["k_cache"].shape[1],
        torch.cuda.current_stream().cuda_stream)
    return st, o, lse


def test_two_calls_in_a_row_match_the_regular_entry_point(built_lib):
    # both cases use several KV splits, i.e. they really go through the built-in scratch
    cases = [W.make_gqa_decode(16, shape_id=31, device="cuda", len_lo=900, len_hi=4000),
             W.make_gqa_decode(5, shape_id=32, device="cuda", lens=[2000, 0, 129, 5000, 777])]
    for a in cases:
        need = built_lib.ako4x_gqa_paged_decode_workspace_bytes(
            a["q"].shape[0], a["kv_indices"].numel(), 1)
        assert 0 < need <= built_lib.ako4x_gqa_paged_decode_noalloc_max_scratch_bytes()
        st, o, lse = _noalloc(a)
        assert st == 0, _cabi.STATUS.get(st, st)
        ro, rlse = gqa_decode.run(*[a[k] for k in KEYS])
        torch.cuda.synchronize()
        assert_close_bf16(o, ro)          # the tolerance of the other GQA tests
        assert_lse_close(lse, rlse)
        assert torch.equal(o, ro) and torch.equal(lse, rlse)  # same kernels: also bit-identical
    # and against the CPU oracle, so that this file does not lean on the regular path's own tests
    a = W.make_gqa_decode(3, shape_id=34, lens=[1500, 3, 4100], extra_pages=9)
    d = W.to_device(a, "cuda")
    st, o, lse = _noalloc(d)
    assert st == 0, _cabi.STATUS.get(st, st)
    ro, rlse = oracle.gqa_paged_decode(*[a[k] for k in KEYS])
    assert_close_bf16(o, ro)
    assert_lse_close(lse, rlse)


def test_oversized_request_is_refused_cleanly(built_lib):
    """A shape whose partials exceed the built-in scratch returns AKO4X_ETOOLARGE before any
    pointer is touched (the pointers below are never dereferenced)."""
    limit = built_lib.ako4x_gqa_paged_decode_noalloc_max_scratch_bytes()
    batch, n_idx = 512, 512 * 8192   # two splits of 512 x 32 heads: about 17 MB of partials
    assert built_lib.ako4x_gqa_paged_decode_workspace_bytes(batch, n_idx, 1) > limit
    a = W.make_gqa_decode(1, shape_id=33, device="cuda", lens=[64])
    st = built_lib.ako4x_gqa_paged_decode_noalloc(
        a["q"].data_ptr(), a["k_cache"].data_ptr(), a["v_cache"].data_ptr(),
        a["kv_indptr"].data_ptr(), a["kv_indices"].data_ptr(), 0.1, a["q"].data_ptr(),
        a["q"].data_ptr(), batch, n_idx, 1, torch.cuda.current_stream().cuda_stream)
    assert st == -5
    torch.cuda.synchronize()
