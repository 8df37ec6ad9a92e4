"""Data-parallel parity on hardware: two ranks through the library against one rank on the concatenated batch
(femtochat_b200/dp_check.py).  Needs two GPUs; on a one-GPU box the test is skipped and the one-GPU emulation in
tests/test_gpu_step.py::test_owner_sharded_update_matches_full_update covers the shard plan."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_ranks_equal_one_rank_on_the_concatenated_batch():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", "-m", "femtochat_b200.dp_check"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert r.returncode == 0 and lines, (r.stdout[-2000:], r.stderr[-2000:])
    out = json.loads(lines[-1])
    assert out["ok"] and out["n_gpus"] == 2
    assert all(c["ok"] and c["nt_exact"] and c["theta_bitwise_replicated"] for c in out["cases"])
