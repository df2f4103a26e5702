"""Entry point of the packed solution for ``moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048``.

``run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor) -> out``: the reference plug-in signature. The work is done by hand-written sm_100a kernels behind
the C ABI of ``ako4x_b200`` (no Triton, no CPU path); the package must be importable where the
solution runs (``pip install -e`` of this repository or its root on ``PYTHONPATH``) with
``ako4x_b200/lib/libako4x_b200.so`` built (``python -m ako4x_b200.build``).
"""
from ako4x_b200.moe import run  # noqa: F401
