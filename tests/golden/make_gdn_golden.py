"""Generates ``gdn_decode_b2.pt`` and ``gdn_decode_b1_nostate.pt``: outputs of the FlashInfer-Bench
definition ``gdn_decode_qk4_v8_d128_k_last`` (flashinfer.trace.templates.gdn, flashinfer-python
0.6.11, run on CPU) on small seeded inputs. Run by hand; the tests only read the files.

    python tests/golden/make_gdn_golden.py
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from ako4x_b200 import workloads as W  # noqa: E402

OUT = Path(__file__).resolve().parent


def main():
    from flashinfer.trace.templates import gdn as G

    for name, batch, with_state in (("gdn_decode_b2", 2, True), ("gdn_decode_b1_nostate", 1, False)):
        a = W.make_gdn_decode(batch, shape_id=900, with_state=with_state)
        o, s = G._gdn_decode_reference(a["q"], a["k"], a["v"], a["state"], a["A_log"], a["a"], a["dt_bias"],
                                       a["b"], a["scale"])
        # the input state (512 KiB per sequence) is not stored: the test regenerates it from the seed
        # and checks this digest of it
        inputs = {k: v for k, v in a.items() if k != "state"}
        inputs["batch"], inputs["shape_id"], inputs["with_state"] = batch, 900, with_state
        if with_state:
            inputs["state_digest"] = a["state"].double().sum().item()
        torch.save({"inputs": inputs, "outputs": {"output": o, "new_state": s}}, OUT / f"{name}.pt")
        print(name, (OUT / f"{name}.pt").stat().st_size // 1024, "KiB")

    # prefill: three packed sequences, one of them empty; only outputs and new states are stored
    lens = [5, 0, 21]
    a = W.make_gdn_prefill(lens, shape_id=900)
    o, s = G._gdn_prefill_reference(a["q"], a["k"], a["v"], a["state"], a["A_log"], a["a"], a["dt_bias"], a["b"],
                                    a["cu_seqlens"], a["scale"])
    torch.save({"inputs": {"seq_lens": lens, "shape_id": 900, "state_digest": a["state"].double().sum().item()},
                "outputs": {"output": o, "new_state": s}}, OUT / "gdn_prefill_s3.pt")
    print("gdn_prefill_s3", (OUT / "gdn_prefill_s3.pt").stat().st_size // 1024, "KiB")


if __name__ == "__main__":
    main()
