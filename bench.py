#!/usr/bin/env python
"""Benchmark of the B200 operator library.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--op moe|gqa_decode|mla_decode] [--ops-only LIST]
                    [--impl ours|reference] [--no-ops-table]

Headline (default ``--op moe``): FP8 block-scale MoE tokens/s at 8192 tokens, 32 local experts per
GPU. With N > 1 (one process per GPU under torchrun) the ranks form an expert-parallel group: the
8192 tokens are sharded 8192/N per rank, every rank owns 32 experts and receives the token rows
routed to them, so the GEMM work per rank is that of the single-GPU call (weak scaling in
(token, expert) pairs). The same run with 8192 tokens PER GPU is reported under
``tokens_per_gpu_8192``, the expert-parallel result is checked against the sum over
``local_expert_offset`` of the single-GPU operator (``ep_parity``), and the decode operators
sharded by batch are timed on the same ranks (``decode_scaling``). ``--op gqa_decode`` /
``mla_decode`` make a decode operator the headline instead. One JSON line is printed by rank 0.

``value`` is measured with the inputs resident in HBM; ``e2e`` is the same metric through the
public Python ``run(...)`` with the step's inputs copied from pinned host memory and the result
copied back inside the timed region. ``roofline`` describes the dominant kernel; ``ops`` lists
microseconds per call and roofline fraction of every operator at its largest configuration
(1 GPU only); ``cpu_baseline`` is the CPU oracle timed on one pass over the same 8192 tokens.

``--impl reference`` times the CPU restatement of the reference operator (the oracle) on the host
cores for the same workload: every step is one pass over all 8192 tokens.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MOE_TOKENS = 8192
FLOP_PER_PAIR_GEMM1 = 2 * 7168 * 4096
FLOP_PER_PAIR_GEMM2 = 2 * 2048 * 7168
FLOP_PER_PAIR = FLOP_PER_PAIR_GEMM1 + FLOP_PER_PAIR_GEMM2


# ---------------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------------
def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm)}


def time_steps(fn, steps, warmup, dist_on, finish=None):
    """W warm-ups, then K steps between two CUDA events on the current stream; max over ranks.
    `finish` (optional) runs before the closing event: a step that uses side streams joins them to
    the current stream there, so the event covers all of its work."""
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    if finish:
        finish()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    if finish:
        finish()
    e1.record()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


_flush_buf = None


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_calls_cold(fn, calls=20, warmup=3):
    """Microseconds per call, each call timed alone after an L2 flush (median, mean)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    us = []
    for _ in range(calls):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        us.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(us), statistics.fmean(us)


def time_call_e2e(fn, step_inputs, calls=10, warmup=2):
    """The same call timed end to end through the plug-in: the per-step inputs (device tensors in
    `step_inputs`, which `fn` reads) are refilled from pinned host copies inside the timed region
    and every output is copied back to pinned host memory. Caches, weights and recurrent states
    stay resident, as they do in a serving engine. Returns (median us, h2d bytes, d2h bytes)."""
    hosts = [pinned(t) for t in step_inputs]
    out = fn()
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    host_outs = [torch.empty(o.shape, dtype=o.dtype, device="cpu", pin_memory=True) for o in outs]
    us = []
    for i in range(warmup + calls):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for d, h in zip(step_inputs, hosts):
            d.copy_(h, non_blocking=True)
        out = fn()
        outs = list(out) if isinstance(out, (tuple, list)) else [out]
        for o, h in zip(outs, host_outs):
            h.copy_(o, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            us.append(e0.elapsed_time(e1) * 1e3)
    h2d = sum(t.numel() * t.element_size() for t in step_inputs)
    d2h = sum(t.numel() * t.element_size() for t in host_outs)
    return statistics.median(us), h2d, d2h


def pinned(t: torch.Tensor) -> torch.Tensor:
    h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
    h.copy_(t)
    return h


# ---------------------------------------------------------------------------------------------
# MoE workload
# ---------------------------------------------------------------------------------------------
MOE_KEYS = ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
            "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
            "routed_scaling_factor"]


def moe_inputs(tokens, rank, device):
    from ako4x_b200 import workloads as W
    a = W.make_moe(tokens, shape_id=rank, device=device, local_expert_offset=32 * rank)
    # the router bias is a model parameter: identical on every rank
    g = torch.Generator(device=device)
    g.manual_seed(W.BASE_SEED + 6999)
    a["routing_bias"] = 0.01 * torch.randn(256, generator=g, device=device, dtype=torch.float32)
    return a


def moe_local_pairs(a, n_ranks_covered=1):
    from ako4x_b200 import moe
    ids, _ = moe.ds_routing(a["routing_logits"], a["routing_bias"], a["routed_scaling_factor"])
    lo = a["local_expert_offset"]
    return int(((ids >= lo) & (ids < lo + 32)).sum().item()), ids


def moe_stage_times(a, calls):
    """Average milliseconds of (route+scatter, GEMM1, GEMM2, combine) from events recorded inside
    the call, on the launching stream."""
    import ctypes
    from ako4x_b200 import _cabi
    L = _cabi.lib()
    tokens = a["hidden_states"].shape[0]
    ws_bytes = L.ako4x_moe_fp8_block_scale_workspace_bytes(tokens, 32)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    out = torch.empty((tokens, 7168), dtype=torch.bfloat16, device="cuda")
    acc = [0.0] * 4
    for _ in range(calls):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        for e in evs:
            e.record()  # creates the underlying handle
        torch.cuda.synchronize()
        arr = (ctypes.c_void_p * 5)(*[e.cuda_event for e in evs])
        st = L.ako4x_moe_fp8_block_scale_staged(
            a["routing_logits"].data_ptr(), a["routing_bias"].data_ptr(), 0,
            a["hidden_states"].data_ptr(), a["hidden_states_scale"].data_ptr(),
            a["gemm1_weights"].data_ptr(), a["gemm1_weights_scale"].data_ptr(),
            a["gemm2_weights"].data_ptr(), a["gemm2_weights_scale"].data_ptr(),
            a["local_expert_offset"], a["routed_scaling_factor"], out.data_ptr(), tokens, 32,
            ws.data_ptr(), ws_bytes, torch.cuda.current_stream().cuda_stream, arr)
        _cabi.check(st, "ako4x_moe_fp8_block_scale_staged")
        torch.cuda.synchronize()
        for i in range(4):
            acc[i] += evs[i].elapsed_time(evs[i + 1])
    return [x / calls for x in acc]


# ---------------------------------------------------------------------------------------------
# per-operator table (1 GPU)
# ---------------------------------------------------------------------------------------------
def ops_table(peaks, calls=15, only=None):
    from ako4x_b200 import (dsa_attention, dsa_indexer, gdn_decode, gdn_prefill, gemm, gqa_decode, mla_decode, mla_prefill, moe,
                            rmsnorm, workloads as W)
    hbm = peaks["hbm_gbs"] * 1e9
    bf16 = peaks["bf16_tflops"] * 1e12
    fp8 = 2 * bf16
    rows = []

    def add(name, cfg, us, bytes_=None, flops=None, bound="hbm", note=None, e2e=None):
        r = {"op": name, "config": cfg, "us_per_call": round(us[0], 2), "us_mean": round(us[1], 2)}
        if e2e is not None:   # host inputs in, outputs back to the host, inside the timed region
            r["e2e_us"] = round(e2e[0], 2)
            r["e2e_h2d_bytes"], r["e2e_d2h_bytes"] = e2e[1], e2e[2]
        if bytes_ is not None:
            r["hbm_gbs"] = round(bytes_ / (us[0] * 1e-6) / 1e9, 1)
            r["hbm_frac"] = round(bytes_ / (us[0] * 1e-6) / hbm, 4)
        if flops is not None:
            peak = fp8 if bound == "tensor_fp8" else bf16
            r["tflops"] = round(flops / (us[0] * 1e-6) / 1e12, 1)
            r["tensor_frac"] = round(flops / (us[0] * 1e-6) / peak, 4)
        r["bound"] = bound
        if note:
            r["note"] = note
        rows.append(r)

    def guarded(name, f):
        try:
            f()
        except Exception as e:  # one failing operator must not hide the others
            rows.append({"op": name, "error": f"{type(e).__name__}: {e}"[:200]})
        torch.cuda.empty_cache()

    def _rms():
        for T in (4096, 520128):
            a = W.make_rmsnorm(T, device="cuda")
            f = lambda: rmsnorm.run(a["hidden_states"], a["weight"])
            us = time_calls_cold(f, calls)
            add("rmsnorm", f"T={T}", us, bytes_=512 * T + 256, e2e=time_call_e2e(f, [a["hidden_states"]]))

    def _gqa():
        for B in (1, 16, 64, 256):
            a = W.make_gqa_decode(B, shape_id=B, device="cuda")
            n = a["kv_indices"].numel()
            f = lambda: gqa_decode.run(a["q"], a["k_cache"], a["v_cache"], a["kv_indptr"], a["kv_indices"],
                                       a["sm_scale"])
            us = time_calls_cold(f, calls)
            add("gqa_decode", f"B={B},sum_len={n}", us, bytes_=4100 * n + 16516 * B, flops=4 * 32 * 128 * n,
                e2e=time_call_e2e(f, [a["q"], a["kv_indptr"], a["kv_indices"]]))
            del a

    def _mla():
        for B in (1, 32, 128):
            a = W.make_mla_decode(B, shape_id=B, device="cuda")
            n = a["kv_indices"].numel()
            f = lambda: mla_decode.run(a["q_nope"], a["q_pe"], a["ckv_cache"], a["kpe_cache"], a["kv_indptr"],
                                       a["kv_indices"], a["sm_scale"])
            us = time_calls_cold(f, calls)
            add("mla_decode", f"B={B},sum_ctx={n}", us, bytes_=1156 * n + B * (16 * 576 * 2 + 16 * 512 * 2 + 64),
                flops=34816 * n, e2e=time_call_e2e(f, [a["q_nope"], a["q_pe"], a["kv_indptr"], a["kv_indices"]]))
            del a

    def _prefill():
        a = W.make_mla_prefill(8, shape_id=0, device="cuda")
        qo, kv = a["qo_indptr"].cpu().long(), a["kv_indptr"].cpu().long()
        ql, kl = qo[1:] - qo[:-1], kv[1:] - kv[:-1]
        pairs = int((ql * (kl - ql) + ql * (ql + 1) // 2).sum())
        f = lambda: mla_prefill.run(a["q_nope"], a["q_pe"], a["ckv_cache"], a["kpe_cache"], a["qo_indptr"],
                                    a["kv_indptr"], a["kv_indices"], a["sm_scale"])
        us = time_calls_cold(f, max(5, calls // 3))
        tq, tkv = int(ql.sum()), int(kl.sum())
        add("mla_prefill", f"batch=8,total_q={tq},total_kv={tkv}", us,
            bytes_=tq * 16 * (576 + 512) * 2 + tkv * 1156, flops=34816 * pairs, bound="tensor_bf16",
            e2e=time_call_e2e(f, [a["q_nope"], a["q_pe"], a["qo_indptr"], a["kv_indptr"], a["kv_indices"]], calls=5))

    def _dsa():
        for T, ctx in ((1, 32768), (64, 32768), (512, 32768)):
            a = W.make_dsa_indexer(T, ctx, shape_id=T, device="cuda")
            args = [a[k] for k in ("q_index_fp8", "k_index_cache_fp8", "weights", "seq_lens", "block_table")]
            us = time_calls_cold(lambda: dsa_indexer.run(*args), calls)
            pages = a["block_table"].shape[1]
            sl = int(a["seq_lens"].long().sum())
            add("dsa_indexer", f"T={T},ctx={ctx}", us,
                bytes_=pages * 8448 + T * (64 * 128 + 64 * 4 + 4 * pages + 2048 * 4),
                flops=2 * 64 * 128 * sl, bound="tensor_fp8",
                e2e=time_call_e2e(lambda: dsa_indexer.run(*args),
                                  [a["q_index_fp8"], a["weights"], a["seq_lens"], a["block_table"]]))
            (idx,) = dsa_indexer.run(*args)
            npages = a["k_index_cache_fp8"].shape[0]
            b = W.make_dsa_attention(T, ctx, idx, npages, shape_id=T, device="cuda")
            f = lambda: dsa_attention.run(b["q_nope"], b["q_pe"], b["ckv_cache"], b["kpe_cache"],
                                          b["sparse_indices"], b["sm_scale"])
            us = time_calls_cold(f, calls)
            nvalid = int((idx >= 0).sum())
            add("dsa_attention", f"T={T},ctx={ctx}", us,
                bytes_=nvalid * 1152 + T * (2048 * 4 + 16 * 1088 * 2 + 64), flops=34816 * nvalid,
                note="gather bytes; served from L2 when rows repeat across tokens",
                e2e=time_call_e2e(f, [b["q_nope"], b["q_pe"], b["sparse_indices"]]))
            del a, b

    def _moe():
        base = W.make_moe(1, shape_id=0, device="cuda")
        for T in (1, 128, 1024, 8192):
            a = W.make_moe(T, shape_id=T % 97, device="cuda", num_local_experts=1)
            for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale"):
                a[k] = base[k]
            pairs, ids = moe_local_pairs(a)
            active = int(torch.unique(ids[(ids >= 0) & (ids < 32)]).numel())
            f = lambda: moe.run(*[a[k] for k in MOE_KEYS])
            us = time_calls_cold(f, max(5, calls // 2))
            add("moe_fp8", f"T={T},local_pairs={pairs},active_experts={active}", us,
                bytes_=active * (44040192 + 10752) + T * (7168 + 224 + 1024 + 14336),
                flops=pairs * FLOP_PER_PAIR, bound="tensor_fp8" if T >= 1024 else "hbm",
                e2e=time_call_e2e(f, [a["routing_logits"], a["hidden_states"], a["hidden_states_scale"]], calls=5))

    def _gdn():
        for B in (1, 16, 64):
            a = W.make_gdn_decode(B, shape_id=B, device="cuda")
            args = [a[k] for k in ("q", "k", "v", "state", "A_log", "a", "dt_bias", "b")]
            us = time_calls_cold(lambda: gdn_decode.run(*args, a["scale"]), calls)
            # end to end the new state stays on the device (it is the next step's input): only the
            # token's output goes back
            add("gdn_decode", f"B={B}", us, bytes_=B * (8 * 2 * 65536 + 2 * 1024 + 2 * 2048 + 32) + 64,
                note="state read + state write",
                e2e=time_call_e2e(lambda: gdn_decode.run(*args, a["scale"])[0], [a["q"], a["k"], a["v"], a["a"], a["b"]]))
            del a

    def _gdnp():
        for lens in ([8192], [4096] * 2, [1024] * 8, [128] * 64):
            a = W.make_gdn_prefill(lens, shape_id=len(lens), device="cuda")
            args = [a[k] for k in ("q", "k", "v", "state", "A_log", "a", "dt_bias", "b", "cu_seqlens")]
            us = time_calls_cold(lambda: gdn_prefill.run(*args, a["scale"]), max(5, calls // 3))
            e2e = time_call_e2e(lambda: gdn_prefill.run(*args, a["scale"])[0],
                                [a["q"], a["k"], a["v"], a["a"], a["b"], a["cu_seqlens"]], calls=5)
            T, n = sum(lens), len(lens)
            add("gdn_prefill", f"seqs={n}x{lens[0]}", us, bytes_=T * (2 * 1024 + 2 * 2048 + 32) + n * 8 * 2 * 65536,
                flops=T * 8 * 128 * 128 * 6, bound="latency",
                note="token-sequential recurrence, rows in parallel; not the chunked form", e2e=e2e)
            del a

    def _gemm():
        for M in (16, 256, 969, 4096, 16294):
            a = W.make_gemm(M, shape_id=M % 89, device="cuda")
            us = time_calls_cold(lambda: gemm.run(a["A"], a["B"]), calls)
            add("gemm_f16", f"M={M},N=2048,K=4096", us, bytes_=2 * (M * 4096 + 2048 * 4096 + M * 2048),
                flops=2 * M * 2048 * 4096, bound="tensor_bf16" if M >= 969 else "hbm",
                e2e=time_call_e2e(lambda: gemm.run(a["A"], a["B"]), [a["A"]]))
            del a

    for name, f in (("rmsnorm", _rms), ("gqa_decode", _gqa), ("mla_decode", _mla), ("mla_prefill", _prefill),
                    ("dsa", _dsa), ("moe_fp8", _moe), ("gdn_decode", _gdn), ("gdn_prefill", _gdnp),
                    ("gemm", _gemm)):
        if only is None or name in only:
            guarded(name, f)
    return rows


# ---------------------------------------------------------------------------------------------
# CPU oracle timing (cpu_baseline and --impl reference)
# ---------------------------------------------------------------------------------------------
def cpu_moe_sample(sample_tokens, steps, warmup):
    """Full-token equivalents/s (local pairs / 8 / time) of the CPU oracle on `sample_tokens`
    tokens of the T=8192 workload."""
    import oracle
    from ako4x_b200 import workloads as W
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    a = W.make_moe(sample_tokens, shape_id=0, device="cpu")
    args = [a[k] for k in MOE_KEYS]
    for _ in range(warmup):
        oracle.moe_fp8_block_scale(*args)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.moe_fp8_block_scale(*args)
    dt = (time.perf_counter() - t0) / max(1, steps)
    ids, _ = oracle.ds_routing(a["routing_logits"], a["routing_bias"], a["routed_scaling_factor"])
    lo = a["local_expert_offset"]
    pairs = int(((ids >= lo) & (ids < lo + 32)).sum())
    return pairs / 8.0 / dt, dt, cores


def cpu_decode_sample(which, batch=4):
    """KV tokens/s of the CPU oracle's decode operator on `batch` sequences of the benchmark's
    length distribution (all host cores)."""
    import oracle
    from ako4x_b200 import workloads as W
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if which == "gqa_decode":
        a = W.make_gqa_decode(batch, shape_id=100, device="cpu", extra_pages=64)
        fn = lambda: oracle.gqa_paged_decode(a["q"], a["k_cache"], a["v_cache"], a["kv_indptr"], a["kv_indices"],
                                             a["sm_scale"])
    else:
        a = W.make_mla_decode(batch, shape_id=100, device="cpu", extra_pages=64)
        fn = lambda: oracle.mla_paged_decode(a["q_nope"], a["q_pe"], a["ckv_cache"], a["kpe_cache"], a["kv_indptr"],
                                             a["kv_indices"], a["sm_scale"])
    n = a["kv_indices"].numel()
    fn()
    t0 = time.perf_counter()
    fn()
    dt = time.perf_counter() - t0
    return n / dt, dt, cores, n


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.op != "moe":
        tps, dt, cores, n = cpu_decode_sample(args.op)
        print(json.dumps({
            "impl": "reference", "metric": f"{args.op}_kv_tokens_per_s", "value": tps, "unit": "kv_tokens/s",
            "n_gpus": args.gpus, "steps": 1, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": f"{args.op} len~U[128/512,8192], page_size=1", "sample_sequences": 4},
            "cpu_baseline": {"value": tps, "unit": "kv_tokens/s", "cores": cores, "kind": "port",
                             "sample": f"4 sequences ({n} KV tokens), one pass of the CPU oracle"},
            "e2e": {"value": tps, "unit": "kv_tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}), flush=True)
        return
    sample = MOE_TOKENS   # the whole workload: a smaller sample is mostly fixed dequantisation cost
    steps = max(1, args.steps)
    warmup = max(0, min(args.warmup, 1))
    tps, dt, cores = cpu_moe_sample(sample, steps, warmup)
    line = {
        "impl": "reference", "metric": "moe_fp8_tokens_per_s", "value": tps,
        "unit": "tokens/s (full-token equivalents: 8 expert applications = 1 token)",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic",
        "config": {"workload": f"moe_fp8_block_scale T={MOE_TOKENS} E_local=32 H=7168 I=2048 (DeepSeek-V3 routing)",
                   "parallelism": "host cores"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s (full-token equivalents)", "cores": cores, "kind": "port",
                         "sample": f"all {MOE_TOKENS} tokens per step (the full workload), 32 local experts"},
        "e2e": {"value": tps, "unit": "tokens/s (full-token equivalents)", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# main arm
# ---------------------------------------------------------------------------------------------
def ep_parity_check(ep, a, world, rows_per_rank=32):
    """Expert-parallel equivalence on the GPUs: for `rows_per_rank` of this rank's tokens the
    expert-parallel output must equal the sum, in rank order, over local_expert_offset = 0, 32, ...
    of the single-GPU operator on the same rows (each rank applies its own experts to every
    rank's sample rows; the bf16 partials are gathered and summed in fp32)."""
    import torch.distributed as dist
    from ako4x_b200 import moe
    T = a["hidden_states"].shape[0]
    n = min(rows_per_rank, T)
    sel = torch.linspace(0, T - 1, n, device="cuda").long()
    out = ep.run(a["routing_logits"], a["routing_bias"], a["hidden_states"], a["hidden_states_scale"],
                 a["gemm1_weights"], a["gemm1_weights_scale"], a["gemm2_weights"], a["gemm2_weights_scale"],
                 a["routed_scaling_factor"])[sel]
    mine = {"lg": a["routing_logits"][sel].contiguous(),
            "x": a["hidden_states"].view(torch.uint8)[sel].contiguous(),
            "xs": a["hidden_states_scale"][:, sel].t().contiguous()}           # [n, 56]
    gathered = {}
    for k, v in mine.items():
        buf = [torch.empty_like(v) for _ in range(world)]
        dist.all_gather(buf, v)
        gathered[k] = torch.cat(buf)                                           # [world*n, ...]
    part = moe.run(gathered["lg"], a["routing_bias"], gathered["x"].view(a["hidden_states"].dtype),
                   gathered["xs"].t().contiguous(), a["gemm1_weights"], a["gemm1_weights_scale"],
                   a["gemm2_weights"], a["gemm2_weights_scale"], a["local_expert_offset"],
                   a["routed_scaling_factor"])                                 # bf16 [world*n, 7168]
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    rank = dist.get_rank()
    ref = torch.zeros((n, 7168), dtype=torch.float32, device="cuda")
    for g in range(world):
        ref += parts[g][rank * n:(rank + 1) * n].float()
    ref = ref.to(torch.bfloat16).float()
    err = (out.float() - ref).abs()
    stats = torch.tensor([float(err.norm()), float(ref.norm()),
                          float((err <= 1e-2 + 1e-2 * ref.abs()).float().mean()),
                          float((ref != 0).any())], device="cuda", dtype=torch.float64)
    allst = [torch.empty_like(stats) for _ in range(world)]
    dist.all_gather(allst, stats)
    allst = torch.stack(allst).cpu()
    fro = float((allst[:, 0].pow(2).sum().sqrt() / allst[:, 1].pow(2).sum().sqrt().clamp(min=1e-30)))
    return {"max_rel_fro": fro, "matched_1e-2": float(allst[:, 2].min()), "rows_per_rank": n,
            "nonzero_reference_on_every_rank": bool(allst[:, 3].min() > 0),
            "ok": bool(fro <= 1e-3 and allst[:, 2].min() >= 0.999 and allst[:, 3].min() > 0)}


def moe_measure(T, args, rank, world, dist_on, with_parity=False):
    """Times the MoE step with `T` tokens on this rank (device-resident, then end to end)."""
    from ako4x_b200 import moe
    a = moe_inputs(T, rank, "cuda")
    ep = None
    if world > 1:
        from ako4x_b200 import moe_ep
        ep = moe_ep.ExpertParallelMoE(rank, world)
        step = lambda: ep.run(a["routing_logits"], a["routing_bias"], a["hidden_states"],
                              a["hidden_states_scale"], a["gemm1_weights"], a["gemm1_weights_scale"],
                              a["gemm2_weights"], a["gemm2_weights_scale"], a["routed_scaling_factor"])
        launches_per_step = ep.kernels_per_step
    else:
        step = lambda: moe.run(*[a[k] for k in MOE_KEYS])
        launches_per_step = 6  # routing, scatter, permute, GEMM1, GEMM2, combine
    with ClockSampler(torch.cuda.current_device()) as cs:
        ms = time_steps(step, args.steps, args.warmup, dist_on)
    clocks = cs.summary()
    # Work done per step: (token, expert) pairs whose expert is owned by a participating rank.
    # A token is fully processed after 8 expert applications, so value = pairs / 8 / time
    # ("full-token equivalents"): with N ranks covering 32*N of the 256 experts it grows with N,
    # and at N = 8 it equals plain tokens/s. Plain tokens-in-flight/s is reported beside it.
    ids, _ = moe.ds_routing(a["routing_logits"], a["routing_bias"], a["routed_scaling_factor"])
    if world > 1:
        pairs_t = (ids < 32 * world).sum().to(torch.int64)
        import torch.distributed as dist
        dist.all_reduce(pairs_t)
    else:
        lo = a["local_expert_offset"]
        pairs_t = ((ids >= lo) & (ids < lo + 32)).sum().to(torch.int64)
    total_pairs = int(pairs_t.item())
    value = total_pairs / 8.0 * args.steps / (ms * 1e-3)
    tokens_in_flight = world * T * args.steps / (ms * 1e-3)

    # end to end: pinned host inputs -> device, run, result -> pinned host, EVERY step. The three
    # legs of consecutive steps overlap (copy-in stream, compute stream, copy-out stream,
    # double-buffered device inputs and host outputs): the serving pattern for a stream of batches.
    h_in = {k: pinned(a[k]) for k in ("routing_logits", "hidden_states", "hidden_states_scale")}
    d_in = [{k: torch.empty_like(a[k]) for k in h_in} for _ in range(2)]
    h_out = [torch.empty((T, 7168), dtype=torch.bfloat16, pin_memory=True) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    counter = [0]

    def e2e_step():
        j = counter[0] & 1
        counter[0] += 1
        cur = torch.cuda.current_stream()
        s_in.wait_event(ev_run[j])          # the step two back has consumed this input buffer
        with torch.cuda.stream(s_in):
            for k in h_in:
                d_in[j][k].copy_(h_in[k], non_blocking=True)
            ev_in[j].record(s_in)
        cur.wait_event(ev_in[j])
        b = dict(a)
        b.update(d_in[j])
        if ep is not None:
            o = ep.run(b["routing_logits"], b["routing_bias"], b["hidden_states"], b["hidden_states_scale"],
                       b["gemm1_weights"], b["gemm1_weights_scale"], b["gemm2_weights"],
                       b["gemm2_weights_scale"], b["routed_scaling_factor"])
        else:
            o = moe.run(*[b[k] for k in MOE_KEYS])
        ev_run[j].record(cur)
        s_out.wait_event(ev_run[j])
        with torch.cuda.stream(s_out):
            h_out[j].copy_(o, non_blocking=True)
            ev_out[j].record(s_out)
        o.record_stream(s_out)

    def e2e_finish():
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)

    e2e_ms = time_steps(e2e_step, args.steps, min(args.warmup, 3), dist_on, finish=e2e_finish)
    h2d = sum(v.numel() * v.element_size() for v in h_in.values())
    d2h = h_out[0].numel() * h_out[0].element_size()
    res = {"T": T, "ms": ms, "e2e_ms": e2e_ms, "pairs": total_pairs, "value": value,
           "tokens_in_flight": tokens_in_flight, "e2e_value": total_pairs / 8.0 * args.steps / (e2e_ms * 1e-3),
           "h2d": h2d, "d2h": d2h, "clocks": clocks, "launches_per_step": launches_per_step, "inputs": a}
    if with_parity and ep is not None:
        res["ep_parity"] = ep_parity_check(ep, a, world)
    if ep is not None:
        res["ep_backend"] = getattr(ep, "backend", "nccl")
        ep.close()
    return res


def traffic_record():
    """DRAM bytes per GEMM1 launch from the last ncu capture of this workload (a small JSON kept
    beside the capture's summary; null when absent)."""
    f = ROOT / "profiles" / "moe_gemm1_T8192_dram_traffic.json"
    try:
        return json.loads(f.read_text())
    except (OSError, ValueError):
        return None


def run_moe(args, rank, world, dist_on, peaks):
    if args.tokens % world:
        raise SystemExit("--tokens must be a multiple of the number of GPUs")
    T = args.tokens // world
    m = moe_measure(T, args, rank, world, dist_on, with_parity=True)
    a = m.pop("inputs")
    line = {
        "metric": "moe_fp8_tokens_per_s", "value": m["value"],
        "unit": "tokens/s (full-token equivalents: 8 expert applications = 1 token)", "n_gpus": world,
        "tokens_in_flight_per_s": m["tokens_in_flight"], "pairs_per_step": m["pairs"],
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": m["ms"] / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3",
        "data": "synthetic",
        "config": {"workload": f"moe_fp8_block_scale T={args.tokens} tokens in the job ({T} per GPU), "
                               "E_local=32 per GPU, H=7168, I=2048, DeepSeek-V3 routing (256 experts, top-8)",
                   "parallelism": f"ep{world}" if world > 1 else "single",
                   "scaling_note": "every rank computes the (token, expert) pairs of its 32 experts over all "
                                   f"{args.tokens} tokens: per-GPU work is fixed as N grows",
                   "l2": "inputs larger than L2 (1.4 GB of expert weights per step)"},
        "clocks": m["clocks"],
        "e2e": {"value": m["e2e_value"], "unit": "tokens/s (full-token equivalents)",
                "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["d2h"]},
        "gpu_launches": m["launches_per_step"] * args.steps,
    }
    if "ep_parity" in m:
        line["ep_parity"] = m["ep_parity"]
        line["ep_backend"] = m["ep_backend"]
    if rank == 0 and world == 1:
        pairs = m["pairs"]
        st = moe_stage_times(a, calls=5)
        fp8_peak = 2 * peaks["bf16_tflops"]
        achieved = pairs * FLOP_PER_PAIR_GEMM1 / (st[1] * 1e-3) / 1e12
        tr = traffic_record() if args.tokens == MOE_TOKENS else None
        line["roofline"] = {
            "bound": "tensor", "kernel": "moe_gemm_tc_kernel<1> (GEMM1 + SwiGLU + two-piece e4m3 h)",
            "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
            "traffic": tr["dram_bytes_per_launch"] if tr else None,
            "traffic_source": ({k: tr[k] for k in ("captured_at_commit", "captured_on", "command") if k in tr}
                               if tr else None),
            "traffic_unit": "bytes per launch (algorithmic: 939.5 MB of W13 + 58 MB activations + 66 MB h)",
            "peak_source": f"2 x {peaks['source']} bf16 burst (no FP8 peak is recorded)",
            "local_pairs": pairs,
            "stage_ms": {"route_scatter": st[0], "gemm1": st[1], "gemm2": st[2], "combine": st[3]},
            "gemm2_achieved_tflops": pairs * FLOP_PER_PAIR_GEMM2 / (st[2] * 1e-3) / 1e12,
        }
    del a
    torch.cuda.empty_cache()
    if world > 1 and not args.no_per_gpu_run:
        # the larger job: 8192 tokens on EVERY GPU (8x the pairs per rank at N = 8)
        g = moe_measure(args.tokens, args, rank, world, dist_on)
        g.pop("inputs")
        torch.cuda.empty_cache()
        line["tokens_per_gpu_8192"] = {
            "tokens_per_gpu": args.tokens, "value": g["value"], "ms_per_step": g["ms"] / args.steps,
            "pairs_per_step": g["pairs"], "e2e_value": g["e2e_value"],
            "tokens_in_flight_per_s": g["tokens_in_flight"]}
    if not args.no_decode_scaling:
        line["decode_scaling"] = []
        for which in ("gqa_decode", "mla_decode"):
            d = run_decode(args, rank, world, dist_on, peaks, which, e2e=False)
            line["decode_scaling"].append({
                "op": which, "kv_tokens_per_s": d["value"], "ms_per_step": d["ms_per_step"],
                "workload": d["config"]["workload"], "hbm_frac_per_gpu": d["roofline"]["frac"]})
            torch.cuda.empty_cache()
    if "ep_parity" in line and not line["ep_parity"]["ok"]:
        line["error"] = "expert-parallel output differs from the sum of single-GPU operators"
    return line


def run_decode(args, rank, world, dist_on, peaks, which, e2e=True):
    from ako4x_b200 import gqa_decode, mla_decode, workloads as W
    if which == "gqa_decode":
        B = 256
        a = W.make_gqa_decode(B, shape_id=100 + rank, device="cuda")
        keys = ["q", "k_cache", "v_cache", "kv_indptr", "kv_indices", "sm_scale"]
        mod, per_tok, hostk = gqa_decode, 4100, ("q", "kv_indptr", "kv_indices")
    else:
        B = 128
        a = W.make_mla_decode(B, shape_id=100 + rank, device="cuda")
        keys = ["q_nope", "q_pe", "ckv_cache", "kpe_cache", "kv_indptr", "kv_indices", "sm_scale"]
        mod, per_tok, hostk = mla_decode, 1156, ("q_nope", "q_pe", "kv_indptr", "kv_indices")
    n = a["kv_indices"].numel()
    tot = torch.tensor([n], device="cuda", dtype=torch.int64)
    if dist_on:
        import torch.distributed as dist
        dist.all_reduce(tot)
    total_tokens = int(tot.item())
    step = lambda: mod.run(*[a[k] for k in keys])
    with ClockSampler(torch.cuda.current_device()) as cs:
        ms = time_steps(step, args.steps, args.warmup, dist_on)
    value = total_tokens * args.steps / (ms * 1e-3)
    if not e2e:
        us = ms / args.steps * 1e3
        achieved = per_tok * n / (us * 1e-6) / 1e9
        return {"value": value, "ms_per_step": ms / args.steps,
                "config": {"workload": f"{which} B={B} per GPU, len~U[128/512,8192], page_size=1"},
                "roofline": {"frac": achieved / peaks["hbm_gbs"]}}
    h_in = {k: pinned(a[k]) for k in hostk}
    d_in = {k: torch.empty_like(a[k]) for k in hostk}
    o0, l0 = step()
    h_o = torch.empty(o0.shape, dtype=o0.dtype, pin_memory=True)
    h_l = torch.empty(l0.shape, dtype=l0.dtype, pin_memory=True)

    def e2e_step():
        for k in h_in:
            d_in[k].copy_(h_in[k], non_blocking=True)
        b = dict(a)
        b.update(d_in)
        o, l = mod.run(*[b[k] for k in keys])
        h_o.copy_(o, non_blocking=True)
        h_l.copy_(l, non_blocking=True)

    e2e_ms = time_steps(e2e_step, args.steps, min(args.warmup, 3), dist_on)
    us = ms / args.steps * 1e3
    achieved = per_tok * n / (us * 1e-6) / 1e9
    return {
        "metric": f"{which}_kv_tokens_per_s", "value": value, "unit": "kv_tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"{which} B={B} per GPU, len~U[128/512,8192], page_size=1",
                   "parallelism": f"batch-sharded x{world}", "l2": "inputs larger than L2 (KV cache of GBs)"},
        "clocks": cs.summary(),
        "e2e": {"value": total_tokens * args.steps / (e2e_ms * 1e-3), "unit": "kv_tokens/s",
                "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in h_in.values()),
                "d2h_bytes_per_step": h_o.numel() * h_o.element_size() + h_l.numel() * 4,
                "note": "the KV cache is resident state; q and the page lists are the step's inputs"},
        # GQA at this size runs in work-list mode: plan + decode + merge; MLA: decode + merge
        "gpu_launches": (3 if which == "gqa_decode" else 2) * args.steps,
        "roofline": {"bound": "hbm", "kernel": f"{which} split kernel + merge", "achieved": achieved,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": None, "peak_source": peaks["source"]},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--op", default="moe", choices=["moe", "gqa_decode", "mla_decode"])
    ap.add_argument("--tokens", type=int, default=MOE_TOKENS,
                    help="MoE tokens in the job (default: the benchmark configuration, 8192), sharded over the GPUs")
    ap.add_argument("--no-per-gpu-run", action="store_true",
                    help="with N > 1, skip the second run with --tokens tokens on every GPU")
    ap.add_argument("--no-decode-scaling", action="store_true",
                    help="skip the batch-sharded decode timings attached to the MoE line")
    ap.add_argument("--no-ops-table", action="store_true")
    ap.add_argument("--ops-only", default=None,
                    help="comma list of rmsnorm,gqa_decode,mla_decode,mla_prefill,dsa,moe_fp8,gdn_decode,gdn_prefill,gemm: time only these "
                         "operators (cold L2) and print their table; used for per-kernel profiles")
    ap.add_argument("--calls", type=int, default=15, help="timed calls per operator row of the table")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local_rank)
    dist_on = world > 1
    if dist_on:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    args.warmup = max(args.warmup, 3)
    peaks = load_peaks()

    from ako4x_b200 import _cabi
    _cabi.lib()  # fail loudly when the CUDA library is missing

    if args.ops_only:
        if world != 1:
            raise SystemExit("--ops-only is a single-GPU mode")
        print(json.dumps({"ops": ops_table(peaks, calls=args.calls, only=set(args.ops_only.split(",")))}), flush=True)
        return
    if args.op == "moe":
        line = run_moe(args, rank, world, dist_on, peaks)
    else:
        line = run_decode(args, rank, world, dist_on, peaks, args.op)

    if rank == 0 and world == 1:
        if not args.no_ops_table:
            torch.cuda.empty_cache()
            line["ops"] = ops_table(peaks)
        if not args.no_cpu_baseline and args.op == "moe":
            tps, dt, cores = cpu_moe_sample(MOE_TOKENS, 1, 0)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s (full-token equivalents)", "cores": cores, "kind": "port",
                                    "sample": f"all {MOE_TOKENS} tokens (the full workload), one pass of the CPU "
                                              f"oracle ({dt:.1f} s), 32 local experts"}
        elif not args.no_cpu_baseline:
            tps, dt, cores, n = cpu_decode_sample(args.op)
            line["cpu_baseline"] = {"value": tps, "unit": "kv_tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"4 sequences ({n} KV tokens), one pass of the CPU oracle ({dt:.1f} s)"}
    if dist_on:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if line.get("error"):
        raise SystemExit(line["error"])


if __name__ == "__main__":
    main()
