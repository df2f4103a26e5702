"""bf16 RMSNorm, hidden size 128.

Same signature as the reference plug-in ``run(hidden_states, weight)``
(reference/rmsnorm-h128/variants/triton_tiered_rows/kernel.py:261-278).
"""
import torch

from . import _cabi


@torch.no_grad()
def run(hidden_states: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if hidden_states.dim() != 2 or hidden_states.shape[1] != 128:
        raise _cabi.Ako4xError("rmsnorm: hidden_states must be [rows, 128]")
    if hidden_states.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise _cabi.Ako4xError("rmsnorm: bf16 tensors expected")
    if weight.numel() != 128:
        raise _cabi.Ako4xError("rmsnorm: weight must have 128 elements")
    x = hidden_states.contiguous()
    out = torch.empty_like(x)
    st = _cabi.lib().ako4x_rmsnorm_h128(_cabi.ptr(x), _cabi.ptr(weight.contiguous()),
                                        _cabi.ptr(out), x.shape[0], _cabi.stream())
    _cabi.check(st, "ako4x_rmsnorm_h128")
    return out
