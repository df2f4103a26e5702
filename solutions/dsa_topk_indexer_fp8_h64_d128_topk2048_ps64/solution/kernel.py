"""Entry point of the packed solution for ``dsa_topk_indexer_fp8_h64_d128_topk2048_ps64``.

``run(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table) -> (topk_indices,)``: the reference plug-in signature. The work is done by hand-written sm_100a kernels behind
the C ABI of ``ako4x_b200`` (no Triton, no CPU path); the package must be importable where the
solution runs (``pip install -e`` of this repository or its root on ``PYTHONPATH``) with
``ako4x_b200/lib/libako4x_b200.so`` built (``python -m ako4x_b200.build``).
"""
from ako4x_b200.dsa_indexer import run  # noqa: F401
