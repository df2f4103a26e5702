"""B200 (sm_100a) kernels for the AKO4X / FlashInfer-Bench operator set.

One module per operator, each exporting ``run(...)`` with the reference plug-in's exact tensor
signature; every ``run`` calls hand-written CUDA through the C ABI in ``include/ako4x_b200.h``.
"""
from . import _cabi  # noqa: F401

__all__ = [
    "rmsnorm", "gqa_decode", "mla_decode", "mla_prefill", "dsa_indexer", "dsa_attention", "moe",
    "gdn_decode", "gdn_prefill", "gemm",
]
