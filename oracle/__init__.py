"""CPU oracle of the operator set: TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` import this
package; nothing under ``ako4x_b200`` does. Each function is a PyTorch-on-CPU restatement of one
reference plug-in's arithmetic and cites the reference lines it follows.
"""
from .rmsnorm import rmsnorm  # noqa: F401
from .attention import (  # noqa: F401
    gqa_paged_decode, mla_paged_decode, mla_paged_prefill, dsa_sparse_attention)
from .indexer import dsa_index_scores, dsa_topk_select, dsa_topk_indexer, unpack_index_cache  # noqa: F401
from .moe import ds_routing, moe_fp8_block_scale  # noqa: F401
from .quantize import fp8_quantize_1x128, index_k_cache_write  # noqa: F401
from .gdn import gdn_decode, gdn_prefill  # noqa: F401
from .gemm import gemm_nt  # noqa: F401
