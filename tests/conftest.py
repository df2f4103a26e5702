import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def built_lib():
    """Builds (or reuses) the shared library; a missing nvcc with no prebuilt library fails."""
    from ako4x_b200 import _cabi, build
    try:
        build.build()
    except RuntimeError:
        if not _cabi.LIB_PATH.exists():
            raise
    return _cabi.lib()


def load_golden(name):
    return torch.load(GOLDEN / f"{name}.pt", weights_only=True)


def assert_close_bf16(out, ref, atol=1e-2, rtol=1e-2, what="output"):
    """|out - ref| <= atol + rtol * |ref| on every element (the reference harness's rule)."""
    out = out.float().cpu()
    ref = ref.float().cpu()
    assert out.shape == ref.shape, f"{what}: shape {tuple(out.shape)} vs {tuple(ref.shape)}"
    err = (out - ref).abs()
    tol = atol + rtol * ref.abs()
    bad = err > tol
    assert not bad.any(), (f"{what}: {int(bad.sum())}/{bad.numel()} elements out of tolerance, "
                           f"max abs err {float(err.max()):.4g}")


def assert_lse_close(out, ref, tol=1e-3, what="lse"):
    out = out.float().cpu()
    ref = ref.float().cpu()
    inf_ref = torch.isinf(ref)
    assert torch.equal(torch.isinf(out), inf_ref), f"{what}: -inf pattern differs"
    assert torch.equal(out[inf_ref], ref[inf_ref]), f"{what}: infinities differ in sign"
    if (~inf_ref).any():
        err = (out[~inf_ref] - ref[~inf_ref]).abs()
        lim = tol * (1.0 + ref[~inf_ref].abs())
        assert (err <= lim).all(), f"{what}: max err {float(err.max()):.4g}"
