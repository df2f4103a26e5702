"""CPU oracle (test infrastructure) for bf16 RMSNorm, hidden 128.

Follows reference/rmsnorm-h128/variants/triton_tiered_rows/kernel.py:226-236,272-273: fp32
accumulation of x^2, mean over the 128 columns, + 1e-6, rsqrt, multiply by the fp32 weight, one
cast to bf16. Pinned against flashinfer.trace.templates.norm (fixtures under tests/golden).
"""
import torch


def rmsnorm(hidden_states: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    x = hidden_states.float()
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return ((x * inv) * weight.float()).to(hidden_states.dtype)
