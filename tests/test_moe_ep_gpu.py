"""Expert parallelism on real GPUs: two ranks exchange token rows over NVLink peer memory and the
result must equal the sum over local_expert_offset of the single-GPU operator (the check bench.py
makes after its timed region). Skipped on boxes with fewer than two GPUs."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("tokens", [8192, 514])
def test_two_rank_exchange_equals_sum_of_single_gpu_operators(built_lib, tokens):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "bench.py"), "--gpus", "2", "--steps", "3",
           "--warmup", "3", "--tokens", str(tokens), "--no-per-gpu-run", "--no-decode-scaling"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert lines, out.stderr[-2000:]
    line = json.loads(lines[-1])
    assert line["ep_backend"] == "p2p"
    par = line["ep_parity"]
    assert par["ok"], par
    assert par["matched_1e-2"] >= 0.999 and par["max_rel_fro"] <= 1e-3
    assert out.returncode == 0, out.stderr[-2000:]
