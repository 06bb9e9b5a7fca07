"""The sharded path on real GPUs: (b,h) units cut over the ranks, each rank's kernel output checked against
the CPU oracle, shards all-gathered over NCCL and the assembled tensor checked again (bench.py's `verify`).
Needs two visible GPUs; skipped otherwise."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("workload", ["c2", "small_causal"])
def test_two_ranks_shard_verify_and_gather(workload):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29613", os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "2", "--warmup", "3",
           "--workload", workload, "--no-cpu-baseline"]
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0"}
    proc = subprocess.run(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, universal_newlines=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:]
    line = json.loads([ln for ln in proc.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["n_gpus"] == 2 and line["scaling"] == "strong"
    assert line["verify"].startswith("ok") and "gathered over NCCL" in line["verify"]
    assert len(line["per_rank_ms"]) == 2
