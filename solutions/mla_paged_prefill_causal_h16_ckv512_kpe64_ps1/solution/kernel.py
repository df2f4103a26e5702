"""Entry point of the packed solution for ``mla_paged_prefill_causal_h16_ckv512_kpe64_ps1``.

``run(q_nope, q_pe, ckv_cache, kpe_cache, qo_indptr, kv_indptr, kv_indices, sm_scale) -> (o, lse)``: the reference plug-in signature. The work is done by hand-written sm_100a kernels behind
the C ABI of ``ako4x_b200`` (no Triton, no CPU path); the package must be importable where the
solution runs (``pip install -e`` of this repository or its root on ``PYTHONPATH``) with
``ako4x_b200/lib/libako4x_b200.so`` built (``python -m ako4x_b200.build``).
"""
from ako4x_b200.mla_prefill import run  # noqa: F401
