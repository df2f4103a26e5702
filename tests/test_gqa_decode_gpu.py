"""Paged GQA decode parity through the C ABI."""
import pytest
import torch

import oracle
from ako4x_b200 import gqa_decode, workloads as W
from conftest import assert_close_bf16, assert_lse_close, load_golden

pytestmark = pytest.mark.gpu
KEYS = ["q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "sm_scale"]


def _run(a):
    d = W.to_device(a, "cuda")
    return gqa_decode.run(*[d[k] for k in KEYS])


def _check(a):
    o, lse = _run(a)
    ro, rlse = oracle.gqa_paged_decode(*[a[k] for k in KEYS])
    assert_close_bf16(o, ro)
    assert_lse_close(lse, rlse)


def test_golden(built_lib):
    g = load_golden("gqa_decode_b4")
    o, lse = _run(g["inputs"])
    assert_close_bf16(o, g["outputs"]["output"])
    assert_lse_close(lse, g["outputs"]["lse"])


@pytest.mark.parametrize("lens", [[1], [15], [16], [17], [128], [547], [2100],
                                  [0, 1, 0], [40, 0, 300, 7, 1024], [8192]])
def test_ragged_lengths(built_lib, lens):
    _check(W.make_gqa_decode(len(lens), shape_id=sum(lens) % 89, lens=lens, extra_pages=13))


@pytest.mark.parametrize("batch", [1, 16, 64])
def test_config_shapes(built_lib, batch):
    """Benchmark configuration shapes, with lengths capped so the CPU oracle stays fast."""
    _check(W.make_gqa_decode(batch, shape_id=batch, len_lo=128, len_hi=1024 if batch > 1 else 8192))


def test_work_list_mode_ragged(built_lib):
    """A batch large and long enough for the work-list mode (equal chunks per CTA): very long next to
    very short and empty sequences, checked against the oracle for every row."""
    lens = [8192] * 20 + [1, 17, 300, 0, 2049, 255, 256, 257] + [5000, 16, 0, 777] * 5
    assert sum(lens) >= 160 * 1024
    _check(W.make_gqa_decode(len(lens), shape_id=41, lens=lens, extra_pages=29))


def test_page_size_4(built_lib):
    g = torch.Generator().manual_seed(5)
    pages, P = 50, 4
    q = torch.randn(2, 32, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(pages, P, 8, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(pages, P, 8, 128, generator=g).to(torch.bfloat16)
    indptr = torch.tensor([0, 7, 19], dtype=torch.int32)
    idx = torch.randperm(pages, generator=g)[:19].to(torch.int32)
    a = dict(q=q, k_cache=k, v_cache=v, kv_indptr=indptr, kv_indices=idx, sm_scale=0.09)
    _check(a)


def test_full_size_split_invariance(built_lib):
    """B=256 at full lengths: appending a key with logit -> -inf weight changes nothing, and
    lse matches a direct fp32 recomputation on one sampled sequence."""
    a = W.make_gqa_decode(256, shape_id=3, device="cuda")
    o, lse = gqa_decode.run(*[a[k] for k in KEYS])
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    b = 37
    s, e = int(a["kv_indptr"][b]), int(a["kv_indptr"][b + 1])
    rows = a["kv_indices"][s:e].long()
    k = a["k_cache"][rows, 0].float()            # [L, 8, 128]
    v = a["v_cache"][rows, 0].float()
    qb = a["q"][b].float().view(8, 4, 128)
    logits = torch.einsum("hgd,lhd->hgl", qb, k) * a["sm_scale"]
    ref_lse = (torch.logsumexp(logits, -1) / 0.6931471805599453).reshape(32)
    ref_o = torch.einsum("hgl,lhd->hgd", torch.softmax(logits, -1), v).reshape(32, 128)
    assert_lse_close(lse[b], ref_lse)
    assert_close_bf16(o[b], ref_o.to(torch.bfloat16))


def test_full_length_sampled_sequences(built_lib):
    """B = 256 with the configured lengths (128..8192), i.e. the work-list mode at full size: eight
    sampled sequences against the CPU oracle (their cache rows compacted into a small cache)."""
    a = W.make_gqa_decode(256, shape_id=256, device="cuda")
    o, lse = gqa_decode.run(*[a[k] for k in KEYS])
    sel = [0, 1, 50, 99, 128, 200, 254, 255]
    ip = a["kv_indptr"].cpu().long()
    rows, indptr = [], [0]
    for b in sel:
        rows.append(a["kv_indices"][ip[b]:ip[b + 1]].long())
        indptr.append(indptr[-1] + int(ip[b + 1] - ip[b]))
    rows = torch.cat(rows)
    dsel = torch.tensor(sel, device="cuda")
    ro, rlse = oracle.gqa_paged_decode(a["q"][dsel].cpu(), a["k_cache"][rows].cpu(), a["v_cache"][rows].cpu(),
                                       torch.tensor(indptr, dtype=torch.int32),
                                       torch.arange(rows.numel(), dtype=torch.int32), a["sm_scale"])
    assert_close_bf16(o[dsel], ro)
    assert_lse_close(lse[dsel], rlse)


def test_non_contiguous_query(built_lib):
    """q as a strided view: the wrapper's contiguous copy must be alive when the kernel runs."""
    a = W.make_gqa_decode(3, shape_id=17, lens=[300, 1, 2049], extra_pages=7)
    d = W.to_device(a, "cuda")
    wide = torch.zeros((3, 32, 256), dtype=torch.bfloat16, device="cuda")
    wide[..., :128] = d["q"]
    o, lse = gqa_decode.run(wide[..., :128], *[d[k] for k in KEYS[1:]])
    ro, rlse = oracle.gqa_paged_decode(*[a[k] for k in KEYS])
    assert_close_bf16(o, ro)
    assert_lse_close(lse, rlse)


def test_same_buffers_new_contents(built_lib):
    a = W.to_device(W.make_gqa_decode(3, lens=[70, 300, 5], extra_pages=3), "cuda")
    o1, _ = gqa_decode.run(*[a[k] for k in KEYS])
    o1 = o1.clone()
    a["v_cache"].mul_(-1)
    o2, _ = gqa_decode.run(*[a[k] for k in KEYS])
    assert torch.equal(o2, -o1)
