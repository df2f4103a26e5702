"""Dense GEMM (gemm_n2048_k4096) on the GPU against the CPU oracle and the golden fixtures of the
reference expression torch.matmul(A, B.T). Tolerance: fp32 accumulation in another order, one
rounding to fp16 / bf16: |diff| <= one unit in the last place of the output (2e-3 relative for
fp16, 8e-3 for bf16) plus 1e-2 absolute for results near zero."""
import pytest
import torch

import oracle
from ako4x_b200 import _cabi, gemm, workloads as W
from conftest import load_golden

pytestmark = pytest.mark.gpu


def _check(c, ref, rtol):
    assert c.shape == ref.shape and c.dtype == ref.dtype
    err = (c.float() - ref.float()).abs()
    assert (err <= rtol * ref.float().abs() + 1e-2).all(), float(err.max())
    assert (c == ref).float().mean().item() > 0.95


@pytest.mark.parametrize("m", [1, 37, 200])
def test_golden(m):
    g = load_golden(f"gemm_m{m}")
    a = W.make_gemm(m, shape_id=g["inputs"]["shape_id"])
    c = gemm.run(a["A"].cuda(), a["B"].cuda()).cpu()
    _check(c, g["outputs"]["C"], 2e-3)
    assert _cabi.lib().ako4x_gemm_device_status() == 0


# every tile width (32, 128, 256 columns), partial and full row tiles, one row, rows not a multiple of 8
@pytest.mark.parametrize("m", [1, 7, 8, 33, 120, 127, 128, 129, 300, 969, 1500, 2400, 4100])
def test_against_oracle(m):
    a = W.make_gemm(m, shape_id=m)
    c = gemm.run(a["A"].cuda(), a["B"].cuda()).cpu()
    _check(c, oracle.gemm_nt(a["A"], a["B"]), 2e-3)
    assert _cabi.lib().ako4x_gemm_device_status() == 0


def test_unsplit_entry_point_agrees():
    """The entry point without a workspace (no K split) against the oracle, and the split form
    against it: same products, fp32 sums in another grouping."""
    import ctypes
    for m in (5, 200, 700):
        a = W.make_gemm(m, shape_id=50 + m, device="cuda")
        c0 = torch.empty((m, 2048), dtype=torch.float16, device="cuda")
        st = _cabi.lib().ako4x_gemm_f16_nt(_cabi.ptr(a["A"]), _cabi.ptr(a["B"]), _cabi.ptr(c0), m, 2048, 4096, 0,
                                           _cabi.stream())
        assert st == 0
        _check(c0.cpu(), oracle.gemm_nt(a["A"].cpu(), a["B"].cpu()), 2e-3)
        c1 = gemm.run(a["A"], a["B"])
        assert _cabi.lib().ako4x_gemm_workspace_bytes(m, 2048, 4096) > 0
        _check(c1.cpu(), c0.cpu(), 2e-3)
        # too small a workspace is refused before anything runs
        ws = torch.empty(64, dtype=torch.uint8, device="cuda")
        st = _cabi.lib().ako4x_gemm_f16_nt_ws(_cabi.ptr(a["A"]), _cabi.ptr(a["B"]), _cabi.ptr(c0), m, 2048, 4096, 0,
                                              _cabi.ptr(ws), 64, _cabi.stream())
        assert st == -4
    assert _cabi.lib().ako4x_gemm_device_status() == 0


def test_bf16_and_other_shapes():
    a = W.make_gemm(515, shape_id=3, n=1024, k=512, dtype=torch.bfloat16)
    c = gemm.run(a["A"].cuda(), a["B"].cuda()).cpu()
    _check(c, oracle.gemm_nt(a["A"], a["B"]), 8e-3)
    a = W.make_gemm(77, shape_id=4, n=256, k=64)
    c = gemm.run(a["A"].cuda(), a["B"].cuda()).cpu()
    _check(c, oracle.gemm_nt(a["A"], a["B"]), 2e-3)


def test_largest_benchmark_size_sampled_rows():
    """M = 16 294 (the largest recorded workload): 96 sampled rows against the oracle, and linearity
    (A and 2A give C and 2C exactly: scaling by two is exact in fp32 and in fp16 away from overflow
    and from the subnormal range, which a few results near zero fall into)."""
    a = W.make_gemm(16294, shape_id=0, device="cuda")
    a["A"].mul_(0.25)
    c = gemm.run(a["A"], a["B"])
    rows = torch.randperm(16294, generator=torch.Generator().manual_seed(1))[:96]
    ref = oracle.gemm_nt(a["A"][rows.cuda()].cpu(), a["B"].cpu())
    _check(c[rows.cuda()].cpu(), ref, 2e-3)
    c2 = gemm.run(a["A"] * 2, a["B"])
    normal = c.abs() > 1e-3
    assert torch.equal(c2[normal], (c * 2)[normal]) and normal.float().mean().item() > 0.999
    assert _cabi.lib().ako4x_gemm_device_status() == 0


def test_empty_and_errors():
    b = torch.zeros((2048, 4096), dtype=torch.float16, device="cuda")
    c = gemm.run(torch.zeros((0, 4096), dtype=torch.float16, device="cuda"), b)
    assert c.shape == (0, 2048)
    with pytest.raises(_cabi.Ako4xError):
        gemm.run(torch.zeros((4, 4096), dtype=torch.float32, device="cuda"), b)
    with pytest.raises(_cabi.Ako4xError):
        gemm.run(torch.zeros((4, 100), dtype=torch.float16, device="cuda"),
                 torch.zeros((2048, 100), dtype=torch.float16, device="cuda"))
    with pytest.raises(_cabi.Ako4xError):
        gemm.run(torch.zeros((4, 4096), dtype=torch.float16, device="cuda"),
                 torch.zeros((200, 4096), dtype=torch.float16, device="cuda"))
