"""Dense GEMM ``C = A @ B.T`` (definition ``gemm_n2048_k4096``: A [M, 4096], B [2048, 4096], fp16).

``run(A, B) -> C`` is the signature of the reference family (reference/gemm-n2048-k4096/README.md,
whose best implementation is ``torch.matmul(A, B.T)``). fp16 or bf16 operands, fp32 accumulation
on tcgen05 tensor cores, output in the operand type. N must be a multiple of 256, K of 64.
"""
import torch

from . import _cabi


@torch.no_grad()
def run(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[1]:
        raise _cabi.Ako4xError("gemm: A must be [M, K] and B [N, K]")
    if A.dtype != B.dtype or A.dtype not in (torch.float16, torch.bfloat16):
        raise _cabi.Ako4xError("gemm: fp16 or bf16 operands of one type expected")
    m, k = A.shape
    n = B.shape[0]
    a, b = A.contiguous(), B.contiguous()
    c = torch.empty((m, n), dtype=A.dtype, device=A.device)
    lib = _cabi.lib()
    # small and medium M split K over CTAs; the fp32 partial products live in this workspace
    ws_bytes = lib.ako4x_gemm_workspace_bytes(m, n, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=A.device) if ws_bytes else None
    st = lib.ako4x_gemm_f16_nt_ws(_cabi.ptr(a), _cabi.ptr(b), _cabi.ptr(c), m, n, k,
                                  1 if A.dtype == torch.bfloat16 else 0,
                                  _cabi.ptr(ws) if ws is not None else None, ws_bytes, _cabi.stream())
    _cabi.check(st, "ako4x_gemm_f16_nt_ws")
    return c
