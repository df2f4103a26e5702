"""CPU oracle (test infrastructure) for the DSA FP8 top-k indexer.

Score: reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py:527-540 — per query row r
and token t < seq_lens[r]: relu(q[r,h] . k[t]) weighted by w[r,h], summed over the 64 heads, then
multiplied by the token's fp32 scale; token t lives at page block_table[r, t // 64], slot t % 64.
Cache page layout (:562, :621-625): 8448 bytes = 64 x 128 e4m3 values then 64 fp32 scales.
Selection: the 2048 highest fp32 scores, ties to the lower token position (the reference ranks
bf16-rounded scores, :541-546, which is lossy; fp32 ranking is the stricter rule), output as
global slots page*64+slot (:436-448) in ascending token position then -1; seq_len <= 2048 lists
every token (:311-320).

Pinned against outputs of the reference's own GPU kernel (v8_radix_bt256/kernel.py::run, run on a
B200 by tests/golden/make_indexer_reference_golden.py; fixture tests/golden/
dsa_indexer_reference_v8.pt): rows of at most 2048 tokens are identical, longer rows differ from the
reference's set only in slots whose score is a bf16 tie of the 2048-th score (the reference ranks
bf16-rounded scores). tests/golden/dsa_indexer_t3.pt is this oracle's own output and only guards
against regressions.
"""
import torch

PAGE = 64
DIM = 128
PAGE_BYTES = PAGE * DIM + PAGE * 4
TOPK = 2048


def unpack_index_cache(k_index_cache: torch.Tensor):
    """Any view with 8448 bytes per page -> (values fp32 [pages,64,128], scales fp32 [pages,64])."""
    npages = k_index_cache.shape[0]
    raw = k_index_cache.contiguous().view(torch.uint8).reshape(npages, PAGE_BYTES)
    vals = raw[:, : PAGE * DIM].contiguous().view(torch.float8_e4m3fn).reshape(npages, PAGE, DIM).float()
    scales = raw[:, PAGE * DIM:].contiguous().view(torch.float32).reshape(npages, PAGE)
    return vals, scales


def dsa_index_scores(q_index_fp8, k_index_cache, weights, seq_lens, block_table):
    """fp32 scores [rows, max_pages*64]; positions t >= seq_len hold -inf."""
    R = q_index_fp8.shape[0]
    max_pages = block_table.shape[1]
    vals, scales = unpack_index_cache(k_index_cache)
    out = torch.full((R, max_pages * PAGE), -float("inf"), dtype=torch.float32)
    q = q_index_fp8.float()
    for r in range(R):
        sl = int(seq_lens[r])
        if sl <= 0:
            continue
        npg = (sl + PAGE - 1) // PAGE
        pages = block_table[r, :npg].long()
        k = vals[pages].reshape(-1, DIM)                    # [npg*64, 128]
        ks = scales[pages].reshape(-1)
        s = torch.relu(q[r] @ k.T)                          # [64, L]
        sc = (s * weights[r].float().unsqueeze(1)).sum(dim=0) * ks
        out[r, :sl] = sc[:sl]
    return out


def dsa_topk_select(scores, seq_lens, block_table, topk: int = TOPK):
    """Exact selection on given fp32 scores. int32 [rows, topk]."""
    R = scores.shape[0]
    out = torch.full((R, topk), -1, dtype=torch.int32)
    for r in range(R):
        sl = int(seq_lens[r])
        if sl <= 0:
            continue
        if sl <= topk:
            pos = torch.arange(sl)
        else:
            s = scores[r, :sl]
            # descending score, ties to the lower position: stable sort of the negated scores
            order = torch.sort(-s, stable=True).indices[:topk]
            pos = torch.sort(order).values
        slot = block_table[r, (pos // PAGE).long()].long() * PAGE + pos % PAGE
        out[r, : pos.numel()] = slot.to(torch.int32)
    return out


def dsa_topk_indexer(q_index_fp8, k_index_cache, weights, seq_lens, block_table):
    scores = dsa_index_scores(q_index_fp8, k_index_cache, weights, seq_lens, block_table)
    return (dsa_topk_select(scores, seq_lens, block_table),)
