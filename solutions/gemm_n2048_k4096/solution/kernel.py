"""Entry point of the packed solution for ``gemm_n2048_k4096``.

``run(A, B) -> C``: the reference family's signature (C = A @ B.T). The work is done by hand-written sm_100a kernels behind
the C ABI of ``ako4x_b200`` (no Triton, no cuBLAS, no CPU path); the package must be importable where the
solution runs (``pip install -e`` of this repository or its root on ``PYTHONPATH``) with
``ako4x_b200/lib/libako4x_b200.so`` built (``python -m ako4x_b200.build``).
"""
from ako4x_b200.gemm import run  # noqa: F401
