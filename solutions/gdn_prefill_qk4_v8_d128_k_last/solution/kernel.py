"""Entry point of the packed solution for ``gdn_prefill_qk4_v8_d128_k_last``.

``run(q, k, v, state, A_log, a, dt_bias, b, cu_seqlens, scale) -> (output, new_state)``: the reference plug-in signature. The work is done by hand-written sm_100a kernels behind
the C ABI of ``ako4x_b200`` (no Triton, no CPU path); the package must be importable where the
solution runs (``pip install -e`` of this repository or its root on ``PYTHONPATH``) with
``ako4x_b200/lib/libako4x_b200.so`` built (``python -m ako4x_b200.build``).
"""
from ako4x_b200.gdn_prefill import run  # noqa: F401
