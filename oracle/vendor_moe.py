"""Times the vendor FP8 block-scale MoE kernel beside ``ako4x_b200.moe.run`` on identical inputs.

TEST / MEASUREMENT INFRASTRUCTURE ONLY (a competitor column, never a product path). The vendor
kernel is ``flashinfer.fused_moe.trtllm_fp8_block_scale_moe`` (flashinfer-python 0.6.11 with its
``flashinfer_cubin`` package), the kernel that
reference/moe-fp8-block-scale-ds-routing-topk8-ng8-kg4-e32-h7168-i2048/variants/
iter2-direct-cpp-bypass/kernel.py:258-288 wraps with the same constants (256 experts, top-8,
8 groups / 4 kept, DeepSeek-V3 routing, DeepSeek FP8 block scales, unshuffled K-major weights).

Its host-side launcher is JIT-compiled by flashinfer (about 17 minutes of nvcc on a CPU box). Build
it once where nvcc is, into the git-ignored ``oracle/_ref``:

    FLASHINFER_WORKSPACE_BASE=oracle/_ref/flashinfer_ws FLASHINFER_CUDA_ARCH_LIST=10.0a \
        python oracle/vendor_moe.py --build-only

and run on a B200 (the workspace travels with the checkout):

    FLASHINFER_WORKSPACE_BASE=oracle/_ref/flashinfer_ws python oracle/vendor_moe.py --tokens 128,1024,8192

Prints one JSON line per token count: both latencies (CUDA events, cold L2, median of the calls)
and how the two outputs compare.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

KEYS = ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
        "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
        "routed_scaling_factor"]


def build_only():
    from flashinfer.jit.fused_moe import gen_trtllm_gen_fused_moe_sm100_module
    spec = gen_trtllm_gen_fused_moe_sm100_module()
    spec.build(verbose=False)
    print(spec.get_library_path())


def vendor_run(a):
    import flashinfer.fused_moe as F
    return F.trtllm_fp8_block_scale_moe(
        a["routing_logits"], a["routing_bias"], a["hidden_states"], a["hidden_states_scale"],
        a["gemm1_weights"], a["gemm1_weights_scale"], a["gemm2_weights"], a["gemm2_weights_scale"],
        256, 8, 8, 4, 2048, int(a["local_expert_offset"]), a["gemm1_weights"].shape[0],
        float(a["routed_scaling_factor"]), routing_method_type=2, use_shuffled_weight=False,  # DeepSeekV3
        weight_layout=0, do_finalize=True, tune_max_num_tokens=max(8192, a["hidden_states"].shape[0]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--build-only", action="store_true")
    ap.add_argument("--tokens", default="128,1024,8192")
    ap.add_argument("--calls", type=int, default=15)
    args = ap.parse_args()
    if args.build_only:
        build_only()
        return
    import torch
    from ako4x_b200 import moe, workloads as W

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn):
        for _ in range(3):
            out = fn()
        ts = []
        for _ in range(args.calls):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return out, ts[len(ts) // 2], ts[0]

    base = W.make_moe(1, shape_id=0, device="cuda")
    for T in [int(x) for x in args.tokens.split(",")]:
        a = W.make_moe(T, shape_id=T % 97, device="cuda", num_local_experts=1)
        for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale"):
            a[k] = base[k]
        rec = {"tokens": T}
        ours, rec["ako4x_us_median"], rec["ako4x_us_min"] = timed(lambda: moe.run(*[a[k] for k in KEYS]))
        try:
            theirs, rec["vendor_us_median"], rec["vendor_us_min"] = timed(lambda: vendor_run(a))
            if isinstance(theirs, (list, tuple)):
                theirs = theirs[0]
            d = (ours.float() - theirs.float()).abs()
            tol = 1e-2 + 1e-2 * theirs.float().abs()
            rec["within_1e-2"] = round((d <= tol).float().mean().item(), 5)
            rec["rel_frobenius"] = float(d.norm() / theirs.float().norm().clamp_min(1e-30))
        except Exception as e:  # the competitor failing must not hide our own number
            rec["vendor_error"] = f"{type(e).__name__}: {e}"[:300]
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
