"""Records outputs of the REFERENCE's own DSA top-k indexer kernel as golden vectors.

Runs on a B200 (the reference implementation is Triton + inline CUDA, GPU only):

    python oracle/stage_reference.py            # where the reference checkout is mounted
    python tests/golden/make_indexer_reference_golden.py [out.pt]

It imports the staged, unmodified reference file (oracle/_ref/dsa_topk_indexer_v8_radix_bt256/
kernel.py, see oracle/stage_reference.py), calls its ``run(...)`` on the seeded synthetic inputs of
``ako4x_b200.workloads.make_dsa_indexer`` (drawn on the CPU, so the CPU test can redraw the same
bits) and stores, per case, the int32 [rows, 2048] result and a digest of the inputs. The file it
writes is committed as tests/golden/dsa_indexer_reference_v8.pt; tests/test_oracle_golden.py pins
oracle/indexer.py against it. It also times the reference on the benchmark shapes (CUDA events)
and writes those numbers next to the output as JSON.
"""
from __future__ import annotations

import hashlib
import importlib.util
import json
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from ako4x_b200 import workloads as W  # noqa: E402

CASES = [  # (rows, context, shape_id)
    (3, 1500, 201),      # every row at most 2048 tokens: the listing path
    (4, 2049, 202),      # straddles the 2048-token limit
    (4, 8192, 203),
    (4, 32768, 204),
]
KEYS = ["q_index_fp8", "k_index_cache_fp8", "weights", "seq_lens", "block_table"]
REF_FILE = ROOT / "oracle" / "_ref" / "dsa_topk_indexer_v8_radix_bt256" / "kernel.py"


def input_digest(a) -> str:
    h = hashlib.sha256()
    for k in KEYS:
        h.update(a[k].contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def load_reference():
    os.environ["DSA_NO_GRAPH"] = "1"      # eager launches: no pointer-keyed graph cache
    spec = importlib.util.spec_from_file_location("ref_dsa_indexer_v8", REF_FILE)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)          # compiles the inline CUDA radix kernel (about a minute)
    return mod


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "tests" / "golden" / "dsa_indexer_reference_v8.pt"
    ref = load_reference()
    torch.cuda.set_device(0)
    cases = []
    for rows, ctx, sid in CASES:
        a = W.make_dsa_indexer(rows, ctx, shape_id=sid, device="cpu")
        d = W.to_device(a, "cuda")
        (idx,) = ref.run(*[d[k] for k in KEYS])
        torch.cuda.synchronize()
        cases.append({"rows": rows, "ctx": ctx, "shape_id": sid, "input_sha256": input_digest(a),
                      "topk_indices": idx.detach().clone().cpu()})
        print(f"rows={rows} ctx={ctx}: valid per row {(idx >= 0).sum(dim=1).tolist()}")
    torch.save({"source": "reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py::run (DSA_NO_GRAPH=1)",
                "torch": str(torch.__version__), "cases": cases}, out_path)
    print("wrote", out_path)

    # the reference's latency on the benchmark shapes, same box, same inputs as bench.py's table
    timings = []
    for T in (1, 64, 512):
        d = W.make_dsa_indexer(T, 32768, shape_id=T, device="cuda")
        args = [d[k] for k in KEYS]
        for _ in range(3):
            ref.run(*args)
        torch.cuda.synchronize()
        us = []
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        for _ in range(15):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ref.run(*args)
            e1.record()
            torch.cuda.synchronize()
            us.append(e0.elapsed_time(e1) * 1e3)
        us.sort()
        timings.append({"op": "dsa_indexer", "config": f"T={T},ctx=32768", "reference_us_median": us[len(us) // 2]})
        print(timings[-1])
    Path(str(out_path) + ".timings.json").write_text(json.dumps(timings, indent=1))


if __name__ == "__main__":
    main()
