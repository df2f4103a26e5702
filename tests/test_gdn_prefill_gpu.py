"""Gated Delta Net prefill on the GPU against the CPU oracle, the golden fixture of the
FlashInfer-Bench definition and the decode operator. Tolerances: fp32 recurrences in another
summation order (the state within 2e-5 of its largest value after hundreds of steps), bf16 outputs
within two rounding steps."""
import pytest
import torch

import oracle
from ako4x_b200 import gdn_decode, gdn_prefill, workloads as W
from conftest import assert_close_bf16, load_golden

pytestmark = pytest.mark.gpu

KEYS = ("q", "k", "v", "state", "A_log", "a", "dt_bias", "b", "cu_seqlens")


def _run(a, scale="given"):
    args = [a[k].cuda() if a[k] is not None else None for k in KEYS]
    o, s = gdn_prefill.run(*args, a["scale"] if scale == "given" else scale)
    torch.cuda.synchronize()
    return o.cpu(), s.cpu()


def _check(o, s, ref_o, ref_s):
    assert o.shape == ref_o.shape and o.dtype == torch.bfloat16 and s.shape == ref_s.shape
    assert (s - ref_s).abs().max().item() <= 2e-5 * max(ref_s.abs().max().item(), 1e-3)
    assert_close_bf16(o, ref_o, atol=2e-3, rtol=2e-2)
    assert (o == ref_o).float().mean().item() > 0.9


def test_golden():
    g = load_golden("gdn_prefill_s3")
    a = W.make_gdn_prefill(g["inputs"]["seq_lens"], shape_id=g["inputs"]["shape_id"])
    o, s = _run(a)
    _check(o, s, g["outputs"]["output"], g["outputs"]["new_state"])
    assert torch.all(s[1] == 0)


@pytest.mark.parametrize("lens", [[1], [15], [16], [17], [33, 1, 64], [0, 100, 0, 7], [257]])
def test_against_oracle(lens):
    a = W.make_gdn_prefill(lens, shape_id=len(lens) + lens[0])
    o, s = _run(a)
    ro, rs = oracle.gdn_prefill(*[a[k] for k in KEYS], a["scale"])
    _check(o, s, ro, rs)


@pytest.mark.parametrize("lens", [[370], [33], [129], [16], [5], [70, 300], [0, 33], [17, 0]])
def test_both_forms_agree(lens):
    """One or two sequences run in the chunked form (16 tokens per step of the state), more run
    token by token; `_chunked=False` forces the latter. Both against the oracle and each other."""
    a = W.make_gdn_prefill(lens, shape_id=21 + len(lens))
    args = [a[k].cuda() if a[k] is not None else None for k in KEYS]
    o1, s1 = gdn_prefill.run(*args, a["scale"], _chunked=False)
    o2, s2 = gdn_prefill.run(*args, a["scale"])
    ro, rs = oracle.gdn_prefill(*[a[k] for k in KEYS], a["scale"])
    _check(o1.cpu(), s1.cpu(), ro, rs)
    _check(o2.cpu(), s2.cpu(), ro, rs)
    _check(o2.cpu(), s2.cpu(), o1.cpu(), s1.cpu())


def test_no_state_default_scale():
    a = W.make_gdn_prefill([40, 9], shape_id=5, with_state=False)
    o, s = _run(a, scale=None)
    ro, rs = oracle.gdn_prefill(*[a[k] for k in KEYS], None)
    _check(o, s, ro, rs)


def test_prefill_equals_repeated_decode():
    """A sequence run through prefill gives the outputs and the state of its tokens fed one by one
    through the decode operator (both on the GPU): 300 tokens, compared directly."""
    a = W.make_gdn_prefill([300], shape_id=11, device="cuda")
    o, s = gdn_prefill.run(*[a[k] for k in KEYS], a["scale"])
    st = a["state"]
    outs = []
    for t in range(300):
        ot, st = gdn_decode.run(a["q"][t:t + 1].unsqueeze(1), a["k"][t:t + 1].unsqueeze(1), a["v"][t:t + 1].unsqueeze(1),
                                st, a["A_log"], a["a"][t:t + 1].unsqueeze(1), a["dt_bias"], a["b"][t:t + 1].unsqueeze(1),
                                a["scale"])
        outs.append(ot[:, 0])
    od = torch.cat(outs)
    assert (s - st).abs().max().item() <= 2e-5 * st.abs().max().item()
    assert_close_bf16(o.cpu(), od.cpu(), atol=2e-3, rtol=2e-2)


def test_long_sequences_sampled():
    """8 192 tokens in four sequences (the largest recorded size): the last 64 outputs of one
    sequence and its final state against the oracle run on that sequence alone."""
    lens = [4096, 1024, 3000, 72]
    a = W.make_gdn_prefill(lens, shape_id=2, device="cuda")
    o, s = gdn_prefill.run(*[a[k] for k in KEYS], a["scale"])
    t0, t1 = 4096, 4096 + 1024
    one = {k: (a[k][t0:t1].cpu() if k in ("q", "k", "v", "a", "b") else a[k].cpu() if torch.is_tensor(a[k]) else a[k]) for k in KEYS}
    one["state"] = a["state"][1:2].cpu()
    one["cu_seqlens"] = torch.tensor([0, 1024])
    ro, rs = oracle.gdn_prefill(*[one[k] for k in KEYS], a["scale"])
    assert (s[1].cpu() - rs[0]).abs().max().item() <= 5e-5 * rs.abs().max().item()
    assert_close_bf16(o[t1 - 64:t1].cpu(), ro[-64:], atol=2e-3, rtol=2e-2)
