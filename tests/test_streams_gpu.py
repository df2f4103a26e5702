"""Stream contract of the C ABI (the reference: launches must go to the caller's current stream or
they are dropped from CUDA-graph capture, templates/skills/cuda/cuda.md:55-81): operators run on a
side stream, can be captured in a CUDA graph and replayed on new contents of the same buffers, and
can be called from two host threads on two streams at once."""
import threading

import pytest
import torch

import oracle
from ako4x_b200 import gqa_decode, mla_decode, rmsnorm, workloads as W
from conftest import assert_close_bf16, assert_lse_close

pytestmark = pytest.mark.gpu
GKEYS = ["q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "sm_scale"]
DKEYS = ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "kv_indptr", "kv_indices", "sm_scale"]


def test_side_stream(built_lib):
    a = W.make_gqa_decode(4, shape_id=51, lens=[900, 33, 0, 2500], extra_pages=9)
    d = W.to_device(a, "cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        o, lse = gqa_decode.run(*[d[k] for k in GKEYS])
    s.synchronize()
    ro, rlse = oracle.gqa_paged_decode(*[a[k] for k in GKEYS])
    assert_close_bf16(o, ro)
    assert_lse_close(lse, rlse)


def test_graph_capture_and_replay_on_new_contents(built_lib):
    """Captured once, replayed after the inputs were overwritten in place: the replay must compute
    the new result (nothing is cached by pointer, every kernel is inside the capture)."""
    a = W.make_rmsnorm(777, device="cuda")
    b = W.make_mla_decode(5, shape_id=52, device="cuda", lens=[300, 2000, 64, 1, 900], extra_pages=7)
    rmsnorm.run(a["hidden_states"], a["weight"])           # warm-up outside the capture (lazy loading)
    mla_decode.run(*[b[k] for k in DKEYS])
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = rmsnorm.run(a["hidden_states"], a["weight"])
        o, lse = mla_decode.run(*[b[k] for k in DKEYS])
    a["hidden_states"].normal_()
    b["q_nope"].normal_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, rmsnorm.run(a["hidden_states"], a["weight"]))
    o2, lse2 = mla_decode.run(*[b[k] for k in DKEYS])
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    ref = oracle.rmsnorm(a["hidden_states"].cpu(), a["weight"].cpu())
    assert_close_bf16(y, ref)


def test_two_host_threads_two_streams(built_lib):
    cases = [W.make_gqa_decode(6, shape_id=53 + i, lens=[1200, 64, 3000, 17, 555, 2048], extra_pages=5) for i in range(2)]
    dev = [W.to_device(c, "cuda") for c in cases]
    torch.cuda.synchronize()
    results, errors = [None, None], []

    def work(i):
        try:
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                for _ in range(20):
                    out = gqa_decode.run(*[dev[i][k] for k in GKEYS])
            s.synchronize()
            results[i] = out
        except Exception as e:  # surfaced in the main thread
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for i in range(2):
        ro, rlse = oracle.gqa_paged_decode(*[cases[i][k] for k in GKEYS])
        assert_close_bf16(results[i][0], ro)
        assert_lse_close(results[i][1], rlse)
