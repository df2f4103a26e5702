"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark
configurations (they stand in for the recorded FlashInfer-Bench workloads, which are not
available offline). Every generator returns a dict whose tensor entries, in order, are the
positional arguments of the operator's ``run(...)``.

``device='cpu'`` draws from a CPU generator (bit-identical inputs for the CPU oracle and, after a
copy, for the GPU); a CUDA device draws on that device, which is what large benchmark shapes use.
Seeds follow ``20260101 + 1000 * op_id + shape_id``.
"""
from __future__ import annotations

import math

import torch

BASE_SEED = 20260101
OP_IDS = {"rmsnorm": 0, "gqa_decode": 1, "mla_decode": 2, "mla_prefill": 3, "dsa_indexer": 4,
          "dsa_attention": 5, "moe": 6, "gdn_decode": 7, "gemm": 8, "gdn_prefill": 9}

FP8_MAX = 448.0


def _gen(op: str, shape_id: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(BASE_SEED + 1000 * OP_IDS[op] + shape_id)
    return g


def _randn_bf16(shape, g, device):
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)


def _randn_bf16_big(shape, g, device, chunk_rows=1 << 18):
    """randn -> bf16 for tensors too large to hold an fp32 copy of."""
    out = torch.empty(shape, device=device, dtype=torch.bfloat16)
    flat = out.view(shape[0], -1)
    for r0 in range(0, shape[0], chunk_rows):
        r1 = min(shape[0], r0 + chunk_rows)
        flat[r0:r1] = torch.randn((r1 - r0, flat.shape[1]), generator=g, device=device,
                                  dtype=torch.float32).to(torch.bfloat16)
    return out


def _uniform_int(lo, hi, n, g, device):
    return torch.randint(lo, hi + 1, (n,), generator=g, device=device, dtype=torch.int64)


def _paging(lens: torch.Tensor, extra_pages: int, g, device):
    """page_size 1: kv_indices = the first sum(len) entries of a random page permutation."""
    total = int(lens.sum())
    pages = total + extra_pages
    perm = torch.randperm(pages, generator=g, device=device)
    indices = perm[:total].to(torch.int32)
    indptr = torch.zeros(lens.numel() + 1, dtype=torch.int32, device=device)
    indptr[1:] = torch.cumsum(lens, 0).to(torch.int32)
    return pages, indptr, indices


# ---- RMSNorm ------------------------------------------------------------------------------

def make_rmsnorm(rows: int, shape_id: int = 0, device="cpu"):
    g = _gen("rmsnorm", shape_id, device)
    x = _randn_bf16((rows, 128), g, device)
    w = (1.0 + 0.1 * torch.randn(128, generator=g, device=device)).to(torch.bfloat16)
    return {"hidden_states": x, "weight": w}


# ---- paged GQA decode ---------------------------------------------------------------------

def make_gqa_decode(batch: int, shape_id: int = 0, device="cpu", len_lo=128, len_hi=8192,
                    extra_pages=1024, lens=None):
    g = _gen("gqa_decode", shape_id, device)
    if lens is None:
        lens = _uniform_int(len_lo, len_hi, batch, g, device)
    else:
        lens = torch.as_tensor(lens, dtype=torch.int64, device=device)
    pages, indptr, indices = _paging(lens, extra_pages, g, device)
    q = _randn_bf16((batch, 32, 128), g, device)
    k = _randn_bf16_big((pages, 1, 8, 128), g, device)
    v = _randn_bf16_big((pages, 1, 8, 128), g, device)
    return {"q": q, "k_cache": k, "v_cache": v, "kv_indptr": indptr, "kv_indices": indices,
            "sm_scale": 1.0 / math.sqrt(128.0)}


# ---- paged MLA decode / prefill -----------------------------------------------------------

def make_mla_decode(batch: int, shape_id: int = 0, device="cpu", len_lo=512, len_hi=8192,
                    extra_pages=1024, lens=None):
    g = _gen("mla_decode", shape_id, device)
    if lens is None:
        lens = _uniform_int(len_lo, len_hi, batch, g, device)
    else:
        lens = torch.as_tensor(lens, dtype=torch.int64, device=device)
    pages, indptr, indices = _paging(lens, extra_pages, g, device)
    return {"q_nope": _randn_bf16((batch, 16, 512), g, device),
            "q_pe": _randn_bf16((batch, 16, 64), g, device),
            "ckv_cache": _randn_bf16_big((pages, 1, 512), g, device),
            "kpe_cache": _randn_bf16_big((pages, 1, 64), g, device),
            "kv_indptr": indptr, "kv_indices": indices, "sm_scale": 1.0 / math.sqrt(192.0)}


def make_mla_prefill(batch: int = 8, shape_id: int = 0, device="cpu", q_lo=16, q_hi=2048,
                     kv_hi=8192, extra_pages=1024, q_lens=None, kv_lens=None):
    g = _gen("mla_prefill", shape_id, device)
    if q_lens is None:
        q_lens = _uniform_int(q_lo, q_hi, batch, g, device)
        u = torch.rand(batch, generator=g, device=device)
        kv_lens = q_lens + (u * (kv_hi - q_lens + 1).float()).long()   # uniform in [q_len, kv_hi]
        kv_lens = torch.minimum(kv_lens, torch.full_like(kv_lens, kv_hi))
    else:
        q_lens = torch.as_tensor(q_lens, dtype=torch.int64, device=device)
        kv_lens = torch.as_tensor(kv_lens, dtype=torch.int64, device=device)
    pages, kv_indptr, indices = _paging(kv_lens, extra_pages, g, device)
    qo_indptr = torch.zeros(batch + 1, dtype=torch.int32, device=device)
    qo_indptr[1:] = torch.cumsum(q_lens, 0).to(torch.int32)
    tq = int(q_lens.sum())
    return {"q_nope": _randn_bf16((tq, 16, 512), g, device),
            "q_pe": _randn_bf16((tq, 16, 64), g, device),
            "ckv_cache": _randn_bf16_big((pages, 1, 512), g, device),
            "kpe_cache": _randn_bf16_big((pages, 1, 64), g, device),
            "qo_indptr": qo_indptr, "kv_indptr": kv_indptr, "kv_indices": indices,
            "sm_scale": 1.0 / math.sqrt(192.0)}


# ---- DSA indexer + sparse attention -------------------------------------------------------

def quantize_e4m3_rows(x: torch.Tensor):
    """Per-row scale = amax / 448 -> (e4m3 values, fp32 scales)."""
    amax = x.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    scale = amax / FP8_MAX
    return (x / scale).to(torch.float8_e4m3fn), scale.squeeze(-1).float()


def pack_index_cache(k_fp8: torch.Tensor, k_scale: torch.Tensor) -> torch.Tensor:
    """[pages,64,128] e4m3 + [pages,64] fp32 -> uint8 [pages, 8448] (values then scales)."""
    npages = k_fp8.shape[0]
    raw = torch.empty(npages, 8448, dtype=torch.uint8, device=k_fp8.device)
    raw[:, :8192] = k_fp8.reshape(npages, 8192).view(torch.uint8)
    raw[:, 8192:] = k_scale.reshape(npages, 64).contiguous().view(torch.uint8).reshape(npages, 256)
    return raw


def make_dsa_indexer(tokens: int, ctx: int, shape_id: int = 0, device="cpu", extra_pages=16):
    """`tokens` consecutive query rows of one sequence of `ctx` tokens (causal seq_lens)."""
    g = _gen("dsa_indexer", shape_id, device)
    npages_seq = (ctx + 63) // 64
    npages = npages_seq + extra_pages
    q = torch.randn((tokens, 64, 128), generator=g, device=device).to(torch.float8_e4m3fn)
    w = torch.rand((tokens, 64), generator=g, device=device, dtype=torch.float32)
    k = torch.randn((npages, 64, 128), generator=g, device=device)
    k_fp8, k_scale = quantize_e4m3_rows(k)
    cache = pack_index_cache(k_fp8, k_scale)
    perm = torch.randperm(npages, generator=g, device=device)[:npages_seq].to(torch.int32)
    block_table = perm.unsqueeze(0).repeat(tokens, 1).contiguous()
    seq_lens = (ctx - tokens + 1 + torch.arange(tokens, device=device)).to(torch.int32)
    return {"q_index_fp8": q, "k_index_cache_fp8": cache, "weights": w, "seq_lens": seq_lens,
            "block_table": block_table}


def make_dsa_attention(tokens: int, ctx: int, sparse_indices: torch.Tensor, num_pages: int,
                       shape_id: int = 0, device="cpu"):
    """Caches are [pages,64,512/64]; `sparse_indices` int32 [tokens,2048] indexes their rows."""
    g = _gen("dsa_attention", shape_id, device)
    return {"q_nope": _randn_bf16((tokens, 16, 512), g, device),
            "q_pe": _randn_bf16((tokens, 16, 64), g, device),
            "ckv_cache": _randn_bf16_big((num_pages, 64, 512), g, device),
            "kpe_cache": _randn_bf16_big((num_pages, 64, 64), g, device),
            "sparse_indices": sparse_indices.to(device), "sm_scale": 1.0 / math.sqrt(192.0)}


# ---- FP8 block-scale MoE ------------------------------------------------------------------

def quantize_e4m3_blocks(w: torch.Tensor, block: int = 128):
    """[..., N, K] fp32 -> e4m3 values + fp32 scales [..., N/block, K/block] (amax / 448)."""
    *lead, n, k = w.shape
    wb = w.reshape(*lead, n // block, block, k // block, block)
    amax = wb.abs().amax(dim=(-3, -1), keepdim=True).clamp(min=1e-12)
    scale = amax / FP8_MAX
    q = (wb / scale).reshape(*lead, n, k).to(torch.float8_e4m3fn)
    return q, scale.reshape(*lead, n // block, k // block).float()


def make_moe(tokens: int, shape_id: int = 0, device="cpu", num_local_experts=32, hidden=7168,
             inter=2048, local_expert_offset=0, skew: float = 0.0):
    g = _gen("moe", shape_id, device)
    logits = torch.randn((tokens, 256), generator=g, device=device, dtype=torch.float32)
    if skew:
        logits = logits + skew * torch.randn((1, 256), generator=g, device=device)
    bias = 0.01 * torch.randn(256, generator=g, device=device, dtype=torch.float32)
    x = torch.randn((tokens, hidden), generator=g, device=device)
    xb = x.reshape(tokens, hidden // 128, 128)
    amax = xb.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    xs = amax / FP8_MAX
    x_fp8 = (xb / xs).reshape(tokens, hidden).to(torch.float8_e4m3fn)
    x_scale = xs.squeeze(-1).t().contiguous().float()                # [hidden/128, tokens]
    w13 = torch.empty((num_local_experts, 2 * inter, hidden), dtype=torch.float8_e4m3fn, device=device)
    s13 = torch.empty((num_local_experts, 2 * inter // 128, hidden // 128), dtype=torch.float32, device=device)
    w2 = torch.empty((num_local_experts, hidden, inter), dtype=torch.float8_e4m3fn, device=device)
    s2 = torch.empty((num_local_experts, hidden // 128, inter // 128), dtype=torch.float32, device=device)
    for e in range(num_local_experts):
        w13[e], s13[e] = quantize_e4m3_blocks(torch.randn((2 * inter, hidden), generator=g, device=device))
        w2[e], s2[e] = quantize_e4m3_blocks(torch.randn((hidden, inter), generator=g, device=device))
    return {"routing_logits": logits, "routing_bias": bias, "hidden_states": x_fp8,
            "hidden_states_scale": x_scale, "gemm1_weights": w13, "gemm1_weights_scale": s13,
            "gemm2_weights": w2, "gemm2_weights_scale": s2,
            "local_expert_offset": int(local_expert_offset), "routed_scaling_factor": 2.5}


def to_device(args: dict, device) -> dict:
    return {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in args.items()}


# ---- Gated Delta Net decode -----------------------------------------------------------------

def make_gdn_decode(batch: int, shape_id: int = 0, device="cpu", with_state=True):
    """q/k L2-normalised per head (as the model feeds them), decay A in [1, 16], state ~ N(0, 0.25)."""
    g = _gen("gdn_decode", shape_id, device)

    def unit(shape):
        x = torch.randn(shape, generator=g, device=device)
        return (x / x.norm(dim=-1, keepdim=True)).to(torch.bfloat16)

    q, k = unit((batch, 1, 4, 128)), unit((batch, 1, 4, 128))
    v = _randn_bf16((batch, 1, 8, 128), g, device)
    state = 0.5 * torch.randn((batch, 8, 128, 128), generator=g, device=device) if with_state else None
    A_log = torch.log(1.0 + 15.0 * torch.rand(8, generator=g, device=device))
    a = _randn_bf16((batch, 1, 8), g, device)
    dt_bias = torch.randn(8, generator=g, device=device)
    b = _randn_bf16((batch, 1, 8), g, device)
    return {"q": q, "k": k, "v": v, "state": state, "A_log": A_log, "a": a, "dt_bias": dt_bias, "b": b,
            "scale": 1.0 / math.sqrt(128.0)}


# ---- dense GEMM -----------------------------------------------------------------------------

def make_gemm(m: int, shape_id: int = 0, device="cpu", n=2048, k=4096, dtype=torch.float16):
    """A [m, k], B [n, k] ~ N(0, 1): C = A @ B.T has entries of size sqrt(k)."""
    g = _gen("gemm", shape_id, device)
    a = torch.randn((m, k), generator=g, device=device, dtype=torch.float32).to(dtype)
    b = torch.randn((n, k), generator=g, device=device, dtype=torch.float32).to(dtype)
    return {"A": a, "B": b}


# ---- Gated Delta Net prefill ------------------------------------------------------------------

def make_gdn_prefill(seq_lens, shape_id: int = 0, device="cpu", with_state=True):
    """Packed sequences of the given lengths; value distributions as make_gdn_decode."""
    g = _gen("gdn_prefill", shape_id, device)
    lens = torch.as_tensor(seq_lens, dtype=torch.int64)
    T, n = int(lens.sum()), lens.numel()

    def unit(shape):
        x = torch.randn(shape, generator=g, device=device)
        return (x / x.norm(dim=-1, keepdim=True)).to(torch.bfloat16)

    q, k = unit((T, 4, 128)), unit((T, 4, 128))
    v = _randn_bf16((T, 8, 128), g, device)
    state = 0.5 * torch.randn((n, 8, 128, 128), generator=g, device=device) if with_state else None
    A_log = torch.log(1.0 + 15.0 * torch.rand(8, generator=g, device=device))
    a = _randn_bf16((T, 8), g, device)
    dt_bias = torch.randn(8, generator=g, device=device)
    b = _randn_bf16((T, 8), g, device)
    cu = torch.zeros(n + 1, dtype=torch.int64, device=device)
    cu[1:] = torch.cumsum(lens, 0).to(device)
    return {"q": q, "k": k, "v": v, "state": state, "A_log": A_log, "a": a, "dt_bias": dt_bias, "b": b,
            "cu_seqlens": cu, "scale": 1.0 / math.sqrt(128.0)}
