"""Generates ``gemm_m*.pt``: the reference expression of the family ``gemm_n2048_k4096``,
``torch.matmul(A, B.T)`` on fp16 tensors (reference/gemm-n2048-k4096/README.md), evaluated on CPU
on seeded inputs. Only the output is stored (the inputs are regenerated from the seed; a digest of
them is kept). Run by hand; the tests only read the files.

    python tests/golden/make_gemm_golden.py
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from ako4x_b200 import workloads as W  # noqa: E402

OUT = Path(__file__).resolve().parent


def main():
    for m in (1, 37, 200):
        a = W.make_gemm(m, shape_id=900 + m)
        c = torch.matmul(a["A"], a["B"].t())
        torch.save({"inputs": {"m": m, "shape_id": 900 + m, "digest": (a["A"].double().sum() + a["B"].double().sum()).item()},
                    "outputs": {"C": c}}, OUT / f"gemm_m{m}.pt")
        print(m, (OUT / f"gemm_m{m}.pt").stat().st_size // 1024, "KiB")


if __name__ == "__main__":
    main()
