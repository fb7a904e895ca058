"""Sharded trainer on 2 GPUs: NCCL collectives, peer-memory kernels, the GEMM-fused
reduce-scatter and the GEMM-fused all-gather must agree (needs >= 2 GPUs)."""
import json
import os
import subprocess
import sys

import pytest
import torch
from conftest import free_port

pytestmark = pytest.mark.gpu
WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_hsdp_worker.py")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_trainer_backends_agree():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = free_port()
    p = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", str(port), WORKER], capture_output=True, text=True, env=env, timeout=300)
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert p.returncode == 0 and len(lines) == 2, p.stdout[-2000:] + p.stderr[-3000:]
    for r in lines:
        for name in ("peer", "fused", "fused_ag"):
            assert r[name]["grad_rel_err"] < 2e-2, (name, r)
            for a, b in zip(r[name]["losses"], r["ref_losses"]):
                assert abs(a - b) < 2e-2, (name, r)
        assert r["ref_losses"][-1] < r["ref_losses"][0]
