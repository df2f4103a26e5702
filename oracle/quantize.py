"""CPU oracle (test infrastructure) for the producers in front of the operator set.

``fp8_quantize_1x128`` restates reference/moe-fp8-block-scale/variants/fused_routing_v2/
kernel.py:495-503 (the quantisation half of its SwiGLU kernel, which is the rule every e4m3 tensor
of the MoE is made with): per 128 consecutive values scale = amax / 448, or 1.0 when
amax <= 1e-10; q = e4m3(x / scale); scales stored block-major [cols/128, rows].
``index_k_cache_write`` applies the same rule per token (128 values) and writes the page layout of
reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py:562, 621-625 (8448 bytes per page: 64
x 128 e4m3 values, then 64 fp32 scales). Parity unpinned for these two: the reference has no test
vector for them; the quantiser is checked against flashinfer-free first principles (dequantised
error bound, scale rule) and both are bit-compared with the CUDA kernels."""
import torch


def fp8_quantize_1x128(x):
    rows, cols = x.shape
    xb = x.float().reshape(rows, cols // 128, 128)
    amax = xb.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 1e-10, amax / 448.0, torch.ones_like(amax))
    q = (xb / scale).reshape(rows, cols).to(torch.float8_e4m3fn)
    return q, scale.squeeze(-1).t().contiguous()


def index_k_cache_write(k, slot_mapping, cache_bytes):
    """cache_bytes uint8 [pages, 8448], modified in place and returned."""
    q, scale = fp8_quantize_1x128(k)            # [n,128] e4m3, [1,n]
    scale = scale.reshape(-1)
    qb = q.view(torch.uint8)
    for t in range(k.shape[0]):
        slot = int(slot_mapping[t])
        if slot < 0 or slot >= cache_bytes.shape[0] * 64:
            continue
        page, s = divmod(slot, 64)
        cache_bytes[page, s * 128:(s + 1) * 128] = qb[t]
        cache_bytes[page, 8192 + 4 * s: 8192 + 4 * s + 4] = scale[t:t + 1].view(torch.uint8)
    return cache_bytes
