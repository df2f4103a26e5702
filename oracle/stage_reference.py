"""Stages the reference's own GPU implementation of the DSA top-k indexer for use as a checker.

TEST INFRASTRUCTURE ONLY. The reference ships its operators as single Python files (Triton plus
one inline-CUDA kernel), so "building" it means placing the file where a GPU run can import it:

    python oracle/stage_reference.py [/path/to/reference/checkout]

copies reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py, unmodified, into
oracle/_ref/dsa_topk_indexer_v8_radix_bt256/kernel.py. oracle/_ref/ is git-ignored: the
reference's sources are never committed here. tests/golden/make_indexer_reference_golden.py
imports the staged file on a GPU and records its outputs as golden vectors for the CPU oracle.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
STAGED = {
    "dsa_topk_indexer_v8_radix_bt256": "reference/dsa-topk-indexer/variants/v8_radix_bt256/kernel.py",
}


def stage(reference_root: str = "/root/reference") -> list[Path]:
    root = Path(reference_root)
    done = []
    for name, rel in STAGED.items():
        src = root / rel
        if not src.exists():
            continue
        dst = HERE / "_ref" / name / "kernel.py"
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
        done.append(dst)
    return done


if __name__ == "__main__":
    for path in stage(*sys.argv[1:2]):
        print(path)
