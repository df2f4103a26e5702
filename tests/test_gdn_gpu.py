"""Gated Delta Net decode on the GPU against the CPU oracle and the golden fixtures of the
FlashInfer-Bench definition. Tolerances: the new state is fp32 arithmetic in another summation
order (2e-6 of the largest state value); the bf16 output may differ by one rounding step."""
import pytest
import torch

import oracle
from ako4x_b200 import gdn_decode, workloads as W
from conftest import assert_close_bf16, load_golden

pytestmark = pytest.mark.gpu

KEYS = ("q", "k", "v", "state", "A_log", "a", "dt_bias", "b")


def _run(a):
    args = [a[k].cuda() if a[k] is not None else None for k in KEYS]
    o, s = gdn_decode.run(*args, a["scale"])
    torch.cuda.synchronize()
    return o.cpu(), s.cpu()


def _check(o, s, ref_o, ref_s):
    assert o.shape == ref_o.shape and o.dtype == torch.bfloat16
    assert s.shape == ref_s.shape and s.dtype == torch.float32
    assert (s - ref_s).abs().max().item() <= 2e-6 * ref_s.abs().max().item() + 1e-7
    assert_close_bf16(o, ref_o, atol=1e-4, rtol=1e-2)
    assert (o == ref_o).float().mean().item() > 0.97


@pytest.mark.parametrize("name", ["gdn_decode_b2", "gdn_decode_b1_nostate"])
def test_golden(name):
    g = load_golden(name)
    i = g["inputs"]
    a = W.make_gdn_decode(i["batch"], shape_id=i["shape_id"], with_state=i["with_state"])
    o, s = _run(a)
    _check(o, s, g["outputs"]["output"], g["outputs"]["new_state"])


@pytest.mark.parametrize("batch", [1, 3, 4, 8, 16, 17, 32, 48, 64])
def test_against_oracle(batch):
    a = W.make_gdn_decode(batch, shape_id=batch)
    o, s = _run(a)
    ro, rs = oracle.gdn_decode(*[a[k] for k in KEYS], a["scale"])
    _check(o, s, ro, rs)


def test_large_batch_sampled_sequences():
    """9 000 sequences (more (sequence, head) pairs than one grid dimension holds): eight sampled
    sequences against the oracle."""
    B = 9000
    a = W.make_gdn_decode(B, shape_id=3, device="cuda")
    o, s = gdn_decode.run(*[a[k] for k in KEYS], a["scale"])
    pick = torch.tensor([0, 1, 4095, 4096, 8190, 8191, 8192, 8999])
    sub = {k: (a[k][pick.cuda()].cpu() if a[k].shape[0] == B else a[k].cpu()) for k in KEYS}
    ro, rs = oracle.gdn_decode(*[sub[k] for k in KEYS], a["scale"])
    _check(o[pick.cuda()].cpu(), s[pick.cuda()].cpu(), ro, rs)


def test_no_state_and_default_scale():
    a = W.make_gdn_decode(5, shape_id=77, with_state=False)
    args = [a[k].cuda() if a[k] is not None else None for k in KEYS]
    o, s = gdn_decode.run(*args, None)
    o0, s0 = gdn_decode.run(*args, 0.0)
    ro, rs = oracle.gdn_decode(*[a[k] for k in KEYS], None)
    _check(o.cpu(), s.cpu(), ro, rs)
    assert torch.equal(o, o0) and torch.equal(s, s0)


def test_recurrence_over_steps():
    """Twenty decode steps fed back through the state stay on the oracle's trajectory (the state
    decays by g each step, so errors do not grow)."""
    a = W.make_gdn_decode(4, shape_id=5)
    state_gpu, state_cpu = a["state"].cuda(), a["state"]
    for step in range(20):
        n = W.make_gdn_decode(4, shape_id=100 + step)
        args = [n[k] for k in KEYS]
        args[3] = state_cpu
        ro, state_cpu = oracle.gdn_decode(*args, n["scale"])
        gargs = [n[k].cuda() for k in KEYS]
        gargs[3] = state_gpu
        o, state_gpu = gdn_decode.run(*gargs, n["scale"])
    assert (state_gpu.cpu() - state_cpu).abs().max().item() <= 1e-5 * state_cpu.abs().max().item()
    assert_close_bf16(o.cpu(), ro, atol=1e-3, rtol=2e-2)


def test_empty_batch_and_errors():
    a = W.make_gdn_decode(1, shape_id=1)
    e = {k: (a[k][:0].cuda() if k in ("q", "k", "v", "state", "a", "b") else a[k].cuda()) for k in KEYS}
    o, s = gdn_decode.run(*[e[k] for k in KEYS], a["scale"])
    assert o.shape == (0, 1, 8, 128) and s.shape == (0, 8, 128, 128)
    from ako4x_b200._cabi import Ako4xError
    with pytest.raises(Ako4xError):
        gdn_decode.run(a["q"].cuda().float(), *[a[k].cuda() for k in KEYS[1:]], a["scale"])
    with pytest.raises(Ako4xError):
        gdn_decode.run(a["q"].cuda()[:, :, :2], *[a[k].cuda() for k in KEYS[1:]], a["scale"])
