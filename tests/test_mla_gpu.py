"""Paged MLA decode, causal MLA prefill and DSA sparse attention parity through the C ABI."""
import pytest
import torch

import oracle
from ako4x_b200 import dsa_attention, mla_decode, mla_prefill, workloads as W
from conftest import assert_close_bf16, assert_lse_close, load_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean(built_lib):
    """No bounded wait of the attention kernels may have given up, before or after a test."""
    from ako4x_b200 import _cabi
    assert _cabi.lib().ako4x_mla_attention_device_status() == 0
    yield
    assert _cabi.lib().ako4x_mla_attention_device_status() == 0
DKEYS = ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "kv_indptr", "kv_indices", "sm_scale"]
PKEYS = ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "qo_indptr", "kv_indptr", "kv_indices", "sm_scale"]
SKEYS = ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "sparse_indices", "sm_scale"]


def _check(mod, fn, keys, a):
    d = W.to_device(a, "cuda")
    o, lse = mod.run(*[d[k] for k in keys])
    ro, rlse = fn(*[a[k] for k in keys])
    assert_close_bf16(o, ro)
    assert_lse_close(lse, rlse)


# ---- decode ------------------------------------------------------------------------------------
def test_decode_golden(built_lib):
    g = load_golden("mla_decode_b3")
    d = W.to_device(g["inputs"], "cuda")
    o, lse = mla_decode.run(*[d[k] for k in DKEYS])
    assert_close_bf16(o, g["outputs"]["output"])
    assert_lse_close(lse, g["outputs"]["lse"])


@pytest.mark.parametrize("lens", [[1], [63], [64], [65], [129], [1000], [0, 2, 0], [512, 0, 77, 3000],
                                  [8192]])
def test_decode_ragged(built_lib, lens):
    _check(mla_decode, oracle.mla_paged_decode, DKEYS,
           W.make_mla_decode(len(lens), shape_id=sum(lens) % 83, lens=lens, extra_pages=11))


@pytest.mark.parametrize("batch", [1, 32, 128])
def test_decode_config_shapes(built_lib, batch):
    _check(mla_decode, oracle.mla_paged_decode, DKEYS,
           W.make_mla_decode(batch, shape_id=batch, len_lo=512, len_hi=1024 if batch > 1 else 8192))


def _sampled_sequences(a, sel, cache_keys):
    """CPU copy of the sub-problem made of the sequences `sel` of a GPU-resident paged batch: their
    cache rows compacted into a small cache, page lists renumbered."""
    ip = a["kv_indptr"].cpu().long()
    rows, indptr = [], [0]
    for b in sel:
        rows.append(a["kv_indices"][ip[b]:ip[b + 1]].long())
        indptr.append(indptr[-1] + int(ip[b + 1] - ip[b]))
    rows = torch.cat(rows)
    sub = {k: a[k][rows].cpu() for k in cache_keys}
    sub["kv_indptr"] = torch.tensor(indptr, dtype=torch.int32)
    sub["kv_indices"] = torch.arange(rows.numel(), dtype=torch.int32)
    return sub


def test_decode_full_length_sampled_sequences(built_lib):
    """B = 128 with the configured context lengths (512..8192): eight sampled sequences of the
    full-size call against the CPU oracle."""
    a = W.make_mla_decode(128, shape_id=128, device="cuda")
    o, lse = mla_decode.run(*[a[k] for k in DKEYS])
    sel = [0, 17, 31, 64, 77, 100, 126, 127]
    sub = _sampled_sequences(a, sel, ("ckv_cache", "kpe_cache"))
    dsel = torch.tensor(sel, device="cuda")
    ro, rlse = oracle.mla_paged_decode(a["q_nope"][dsel].cpu(), a["q_pe"][dsel].cpu(), sub["ckv_cache"],
                                       sub["kpe_cache"], sub["kv_indptr"], sub["kv_indices"], a["sm_scale"])
    assert_close_bf16(o[dsel], ro)
    assert_lse_close(lse[dsel], rlse)


def test_split_views_as_inputs(built_lib):
    """q_nope / q_pe as the two halves of one [n,16,576] tensor (non-contiguous views): the wrapper's
    contiguous copies must both be alive when the kernel runs."""
    a = W.make_mla_decode(6, shape_id=61, lens=[700, 64, 1, 2500, 130, 999], extra_pages=13)
    d = W.to_device(a, "cuda")
    q = torch.cat([d["q_nope"], d["q_pe"]], dim=-1)
    qn, qp = q.split([512, 64], dim=-1)
    assert not qn.is_contiguous() and not qp.is_contiguous()
    o, lse = mla_decode.run(qn, qp, *[d[k] for k in DKEYS[2:]])
    ro, rlse = oracle.mla_paged_decode(*[a[k] for k in DKEYS])
    assert_close_bf16(o, ro)
    assert_lse_close(lse, rlse)
    # the same through prefill (one query token per sequence, kv_len = its context) and DSA
    qo = torch.arange(7, dtype=torch.int32, device="cuda")
    o2, lse2 = mla_prefill.run(qn, qp, d["ckv_cache"], d["kpe_cache"], qo, d["kv_indptr"], d["kv_indices"],
                               d["sm_scale"])
    assert_close_bf16(o2, ro)
    assert_lse_close(lse2, rlse)


# ---- prefill -----------------------------------------------------------------------------------
def test_prefill_golden(built_lib):
    g = load_golden("mla_prefill_b3")
    d = W.to_device(g["inputs"], "cuda")
    o, lse = mla_prefill.run(*[d[k] for k in PKEYS])
    assert_close_bf16(o, g["outputs"]["output"])
    assert_lse_close(lse, g["outputs"]["lse"])


@pytest.mark.parametrize("q_lens,kv_lens", [([1], [1]), ([16], [16]), ([16], [400]), ([70, 5], [70, 900]),
                                             ([3, 0, 9], [10, 0, 9]), ([130, 64, 1], [200, 64, 333])])
def test_prefill_ragged(built_lib, q_lens, kv_lens):
    _check(mla_prefill, oracle.mla_paged_prefill, PKEYS,
           W.make_mla_prefill(len(q_lens), shape_id=sum(kv_lens) % 79, q_lens=q_lens, kv_lens=kv_lens,
                              extra_pages=9))


@pytest.mark.parametrize("q_lens,kv_lens", [([48], [48]), ([50, 0, 7], [60, 0, 300]), ([200], [2000]),
                                             ([9, 129, 8, 1], [500, 129, 8, 257])])
def test_prefill_tensor_core_path(built_lib, q_lens, kv_lens):
    """48 query tokens and more take the tcgen05 kernel: partial query tiles, empty sequences,
    kv_len == q_len, key tiles that straddle the causal limit."""
    _check(mla_prefill, oracle.mla_paged_prefill, PKEYS,
           W.make_mla_prefill(len(q_lens), shape_id=sum(kv_lens) % 83, q_lens=q_lens, kv_lens=kv_lens,
                              extra_pages=17))


@pytest.mark.parametrize("q_len", [20, 100])
def test_prefill_page_size_4(built_lib, q_len):
    """Pages of four tokens (kv_len = pages x 4), on the small-call kernel and on the tensor-core one."""
    g = torch.Generator().manual_seed(7 + q_len)
    npages, used = 96, 70                       # 280 keys
    a = W.make_mla_prefill(1, shape_id=5, q_lens=[q_len], kv_lens=[used * 4], extra_pages=npages * 4 - used * 4)
    a["ckv_cache"] = a["ckv_cache"][: npages * 4].reshape(npages, 4, 512).contiguous()
    a["kpe_cache"] = a["kpe_cache"][: npages * 4].reshape(npages, 4, 64).contiguous()
    a["kv_indices"] = torch.randperm(npages, generator=g)[:used].to(torch.int32)
    a["kv_indptr"] = torch.tensor([0, used], dtype=torch.int32)
    _check(mla_prefill, oracle.mla_paged_prefill, PKEYS, a)


def test_prefill_config_shape_reduced(built_lib):
    """Batch 8 with the configured distributions at a quarter of the lengths (oracle cost)."""
    _check(mla_prefill, oracle.mla_paged_prefill, PKEYS,
           W.make_mla_prefill(8, shape_id=1, q_lo=16, q_hi=512, kv_hi=2048))


def test_prefill_last_query_equals_decode(built_lib):
    """Full-size property: the last query of every sequence attends to the whole KV list, which
    is exactly a decode call on the same cache."""
    a = W.make_mla_prefill(8, shape_id=2, device="cuda")
    o, lse = mla_prefill.run(*[a[k] for k in PKEYS])
    last = (a["qo_indptr"][1:] - 1).long()
    od, lsed = mla_decode.run(a["q_nope"][last].contiguous(), a["q_pe"][last].contiguous(),
                              a["ckv_cache"], a["kpe_cache"], a["kv_indptr"], a["kv_indices"],
                              a["sm_scale"])
    assert_close_bf16(o[last], od)
    assert_lse_close(lse[last], lsed)
    assert torch.isfinite(lse).all()


def test_prefill_full_size_sampled_queries(built_lib):
    """The full-size batch (8 sequences, about 6 500 query tokens against up to 8 192 keys each):
    24 sampled query tokens, first, last and interior ones, against the CPU oracle. A query at
    position i of a sequence with q_len queries and kv_len keys sees the first kv_len - q_len + i + 1
    keys, so each sample is a one-query oracle problem over a prefix of the sequence's page list."""
    a = W.make_mla_prefill(8, shape_id=2, device="cuda")
    o, lse = mla_prefill.run(*[a[k] for k in PKEYS])
    qo, kv = a["qo_indptr"].cpu().long(), a["kv_indptr"].cpu().long()
    g = torch.Generator().manual_seed(7)
    ckv, kpe, idx = a["ckv_cache"].cpu(), a["kpe_cache"].cpu(), a["kv_indices"].cpu()
    for s in range(8):
        q_len, kv_len = int(qo[s + 1] - qo[s]), int(kv[s + 1] - kv[s])
        picks = {0, q_len - 1, int(torch.randint(0, q_len, (1,), generator=g))}
        for i in picks:
            t = int(qo[s]) + i
            vis = kv_len - q_len + i + 1
            ro, rlse = oracle.mla_paged_prefill(
                a["q_nope"][t:t + 1].cpu(), a["q_pe"][t:t + 1].cpu(), ckv, kpe, torch.tensor([0, 1], dtype=torch.int32),
                torch.tensor([0, vis], dtype=torch.int32), idx[int(kv[s]):int(kv[s]) + vis], a["sm_scale"])
            assert_close_bf16(o[t:t + 1].cpu(), ro)
            assert_lse_close(lse[t:t + 1].cpu(), rlse)


def test_prefill_repeatable_full_size(built_lib):
    """Twenty calls on the full-size ragged batch give bit-identical outputs. The batch has a last
    query tile of 7 tokens, i.e. a softmax warp with masked rows beside three warps on the short
    unmasked path: the warps of one CTA then run a whole key tile apart, which is the timing that
    once let a fast warp's mbarrier arrival stand in for a slow warp's."""
    a = W.make_mla_prefill(8, shape_id=2, device="cuda")
    small = W.make_mla_prefill(3, device="cuda", q_lens=[64, 200, 9], kv_lens=[64, 1000, 500], extra_pages=64)
    o0, lse0 = mla_prefill.run(*[a[k] for k in PKEYS])
    o0, lse0 = o0.clone(), lse0.clone()
    for _ in range(20):
        mla_prefill.run(*[small[k] for k in PKEYS])
        o, lse = mla_prefill.run(*[a[k] for k in PKEYS])
        assert torch.equal(o, o0)
        assert torch.equal(lse, lse0)
    assert torch.isfinite(o0.float()).all()


# ---- DSA sparse attention ----------------------------------------------------------------------
def test_sparse_golden(built_lib):
    g = load_golden("dsa_attention_t4")
    d = W.to_device(g["inputs"], "cuda")
    o, lse = dsa_attention.run(*[d[k] for k in SKEYS])
    assert_close_bf16(o, g["outputs"]["output"])
    assert_lse_close(lse, g["outputs"]["lse"])


@pytest.mark.parametrize("tokens,valid", [(1, 2048), (1, 100), (3, 1500), (64, 2048)])
def test_sparse_against_oracle(built_lib, tokens, valid):
    pages = 40
    g = torch.Generator().manual_seed(tokens * 7 + valid)
    idx = torch.full((tokens, 2048), -1, dtype=torch.int32)
    for t in range(tokens):
        idx[t, :valid] = torch.randperm(pages * 64, generator=g)[:valid].to(torch.int32)
    if tokens > 1:
        idx[1, ::3] = -1  # holes anywhere in the list
    _check(dsa_attention, oracle.dsa_sparse_attention, SKEYS,
           W.make_dsa_attention(tokens, pages * 64, idx, pages, shape_id=tokens))


def test_sparse_order_invariance_full_size(built_lib):
    """T=512 with 2048 indices each: permuting a row's index list must not change its result
    beyond fp32 summation order."""
    pages, T = 512, 512
    g = torch.Generator(device="cuda").manual_seed(11)
    idx = torch.stack([torch.randperm(pages * 64, generator=g, device="cuda")[:2048] for _ in range(8)])
    idx = idx.repeat(T // 8, 1).to(torch.int32)
    a = W.make_dsa_attention(T, pages * 64, idx, pages, shape_id=3, device="cuda")
    o1, l1 = dsa_attention.run(*[a[k] for k in SKEYS])
    a["sparse_indices"] = idx.flip(1).contiguous()
    o2, l2 = dsa_attention.run(*[a[k] for k in SKEYS])
    assert_close_bf16(o2, o1)
    assert_lse_close(l2, l1)
