"""The producers in front of the operator set: the FP8 activation quantiser that makes the MoE's
``hidden_states`` / ``hidden_states_scale`` pair and the writer of the indexer's paged index-K cache
(rule and layouts: reference/moe-fp8-block-scale/variants/fused_routing_v2/kernel.py:495-503 and
reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py:562, 621-625)."""
import torch

from . import _cabi


@torch.no_grad()
def quantize_1x128(x):
    """bf16 [rows, cols] -> (e4m3 [rows, cols], fp32 scales [cols/128, rows]); cols % 128 == 0."""
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.shape[1] % 128:
        raise _cabi.Ako4xError("quantize_1x128: bf16 [rows, cols] with cols a multiple of 128")
    rows, cols = x.shape
    xc = x.contiguous()
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty((cols // 128, rows), dtype=torch.float32, device=x.device)
    st = _cabi.lib().ako4x_fp8_quantize_1x128(_cabi.ptr(xc), _cabi.ptr(q), _cabi.ptr(scale), rows, cols,
                                              _cabi.stream())
    del xc
    _cabi.check(st, "ako4x_fp8_quantize_1x128")
    return q, scale


@torch.no_grad()
def index_k_cache_write(k, slot_mapping, k_index_cache):
    """Stores bf16 index keys [tokens, 128] into the paged cache (any view with 8448 bytes per page) at
    global slots ``slot_mapping`` (int32, page * 64 + slot; -1 skips the token). In place."""
    npages = k_index_cache.shape[0]
    if k.dim() != 2 or k.shape[1] != 128 or k.dtype != torch.bfloat16:
        raise _cabi.Ako4xError("index_k_cache_write: k must be bf16 [tokens, 128]")
    if slot_mapping.dtype != torch.int32 or slot_mapping.numel() != k.shape[0]:
        raise _cabi.Ako4xError("index_k_cache_write: slot_mapping must be int32 [tokens]")
    if k_index_cache.numel() * k_index_cache.element_size() != npages * 8448 or not k_index_cache.is_contiguous():
        raise _cabi.Ako4xError("index_k_cache_write: the cache must be contiguous with 8448 bytes per page")
    kc, sm = k.contiguous(), slot_mapping.contiguous()
    st = _cabi.lib().ako4x_dsa_index_k_cache_write(_cabi.ptr(kc), _cabi.ptr(sm), _cabi.ptr(k_index_cache),
                                                   k.shape[0], npages, _cabi.stream())
    del kc, sm
    _cabi.check(st, "ako4x_dsa_index_k_cache_write")
    return k_index_cache
