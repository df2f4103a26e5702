"""ctypes binding of ``libako4x_b200.so`` (the C ABI declared in ``include/ako4x_b200.h``).

The operators have no CPU path: when the shared library is absent every call raises. Arguments
cross the boundary as raw device pointers, sizes and scalars; the CUDA stream is PyTorch's
current stream, passed as an opaque handle.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libako4x_b200.so"
HEADER_PATH = _PKG.parent / "include" / "ako4x_b200.h"

STATUS = {
    0: "AKO4X_OK",
    -1: "AKO4X_EINVAL",
    -2: "AKO4X_EUNSUPPORTED_SHAPE",
    -3: "AKO4X_ELAUNCH",
    -4: "AKO4X_EWORKSPACE",
    -5: "AKO4X_ETOOLARGE",
}


class Ako4xError(RuntimeError):
    """A C-ABI call returned a negative status."""


_lib = None


def declared_symbols() -> list[str]:
    """Names of every function the public header declares."""
    text = HEADER_PATH.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ako4x_[a-z0-9_]+)\s*\(", text)))


def lib() -> ctypes.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise Ako4xError(
                f"{LIB_PATH} is missing: build it with `python -m ako4x_b200.build` "
                "(the operators have no fallback path)")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _declare(_lib)
    return _lib


_P = ctypes.c_void_p
_I64 = ctypes.c_int64
_I32 = ctypes.c_int32
_F32 = ctypes.c_float
_SZ = ctypes.c_size_t
_INT = ctypes.c_int

_SIGNATURES = {
    "ako4x_abi_version": (_INT, []),
    "ako4x_rmsnorm_h128": (_INT, [_P, _P, _P, _I64, _P]),
    "ako4x_gqa_paged_decode_workspace_bytes": (_SZ, [_I64, _I64, _I64]),
    "ako4x_gqa_paged_decode": (_INT, [_P, _P, _P, _P, _P, _F32, _P, _P, _I64, _I64, _I64, _P, _SZ, _P]),
    "ako4x_gqa_paged_decode_device_status": (_INT, []),
    "ako4x_gqa_paged_decode_noalloc_max_scratch_bytes": (_SZ, []),
    "ako4x_gqa_paged_decode_noalloc": (_INT, [_P, _P, _P, _P, _P, _F32, _P, _P, _I64, _I64, _I64, _P]),
    "ako4x_mla_paged_decode_workspace_bytes": (_SZ, [_I64, _I64, _I64]),
    "ako4x_mla_paged_decode": (_INT, [_P, _P, _P, _P, _P, _P, _F32, _P, _P, _I64, _I64, _I64, _P, _SZ, _P]),
    "ako4x_mla_attention_device_status": (_INT, []),
    "ako4x_mla_paged_prefill_workspace_bytes": (_SZ, [_I64, _I64, _I64, _I64]),
    "ako4x_mla_paged_prefill": (_INT, [_P, _P, _P, _P, _P, _P, _P, _F32, _P, _P, _I64, _I64, _I64, _I64, _P, _SZ, _P]),
    "ako4x_dsa_topk_indexer_workspace_bytes": (_SZ, [_I64, _I64]),
    "ako4x_dsa_topk_indexer": (_INT, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _SZ, _P]),
    "ako4x_dsa_index_scores": (_INT, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "ako4x_dsa_topk_select": (_INT, [_P, _P, _P, _P, _I64, _I64, _P]),
    "ako4x_dsa_indexer_device_status": (_INT, []),
    "ako4x_dsa_sparse_attention_workspace_bytes": (_SZ, [_I64, _I64]),
    "ako4x_dsa_sparse_attention": (_INT, [_P, _P, _P, _P, _P, _F32, _P, _P, _I64, _I64, _I64, _P, _SZ, _P]),
    "ako4x_moe_fp8_block_scale_workspace_bytes": (_SZ, [_I64, _I64]),
    "ako4x_moe_fp8_block_scale": (_INT, [_P, _P, _INT, _P, _P, _P, _P, _P, _P, _I32, _F32, _P, _I64, _I64, _P, _SZ, _P]),
    "ako4x_moe_fp8_block_scale_staged": (_INT, [_P, _P, _INT, _P, _P, _P, _P, _P, _P, _I32, _F32, _P, _I64, _I64, _P, _SZ, _P, _P]),
    "ako4x_moe_fp8_block_scale_status_offset": (_SZ, [_I64]),
    "ako4x_moe_ds_routing": (_INT, [_P, _P, _INT, _F32, _P, _P, _I64, _P]),
    "ako4x_moe_ep_combine": (_INT, [_P, _P, _P, _I64, _I64, _I64, _P]),
    "ako4x_moe_ep_buffer_bytes": (_SZ, [_I64, _I64]),
    "ako4x_moe_ep_workspace_bytes": (_SZ, [_I64, _I64, _I64, _I64]),
    "ako4x_moe_fp8_block_scale_ep": (_INT, [_P, _P, _INT, _P, _P, _P, _P, _P, _P, _F32, _P, _I64, _I64, _I64, _I64,
                                             _I64, _I32, _P, _P, _SZ, _P]),
    "ako4x_moe_ep_status": (_INT, [_P]),
    "ako4x_gemm_f16_nt": (_INT, [_P, _P, _P, _I64, _I64, _I64, _INT, _P]),
    "ako4x_gemm_device_status": (_INT, []),
    "ako4x_gemm_workspace_bytes": (_SZ, [_I64, _I64, _I64]),
    "ako4x_gemm_f16_nt_ws": (_INT, [_P, _P, _P, _I64, _I64, _I64, _INT, _P, _SZ, _P]),
    "ako4x_gdn_prefill": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _F32, _P, _P, _I64, _I64, _P, _SZ, _P]),
    "ako4x_gdn_prefill_workspace_bytes": (_SZ, [_I64, _I64]),
    "ako4x_gdn_decode": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _F32, _P, _P, _I64, _P]),
    "ako4x_fp8_quantize_1x128": (_INT, [_P, _P, _P, _I64, _I64, _P]),
    "ako4x_dsa_index_k_cache_write": (_INT, [_P, _P, _P, _I64, _I64, _P]),
    "ako4x_dsa_indexer_attention_workspace_bytes": (_SZ, [_I64, _I64]),
    "ako4x_dsa_indexer_attention": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _F32, _P, _P, _P, _I64, _I64, _I64,
                                            _P, _SZ, _P]),
}


def _declare(l: ctypes.CDLL) -> None:
    for name, (res, args) in _SIGNATURES.items():
        try:
            fn = getattr(l, name)
        except AttributeError:
            continue  # reported by the symbol test; calling it raises AttributeError
        fn.restype = res
        fn.argtypes = args


def check(status: int, what: str) -> None:
    if status != 0:
        raise Ako4xError(f"{what} failed: {STATUS.get(status, status)}")


def ptr(t: torch.Tensor | None) -> int | None:
    """Device address of a contiguous CUDA tensor (None stays a null pointer)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise Ako4xError("ako4x_b200 operators take CUDA tensors only (there is no CPU path)")
    if not t.is_contiguous():
        raise Ako4xError("tensor must be contiguous")
    return t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def workspace(nbytes: int, device) -> torch.Tensor | None:
    """Scratch from PyTorch's caching allocator; contents are undefined."""
    if nbytes <= 0:
        return None
    return torch.empty(int(nbytes), dtype=torch.uint8, device=device)
