"""Fault tolerance on real GPUs (needs >= 2): two replica groups, one GPU each, gradients
averaged by ProcessGroupB200's peer-memory allreduce.  Replica 1 leaves between steps; the
survivor learns of it on the host (heartbeat expiry -> new quorum -> team rebuilt for a world
of one) before its next launch, keeps training, and the restarted replica heals over NVLink
(P2PTransport).  NVLS is disabled and no kernel of a leaving rank is ever in flight."""
import json
import os
import subprocess
import sys
import time

import pytest
import torch

from torchft_b200._ftcp import LighthouseServer

pytestmark = pytest.mark.gpu
WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ft_gpu_worker.py")


def _spawn(replica, gpu, lighthouse, steps, exit_at=-1):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    return subprocess.Popen(
        [sys.executable, WORKER, "--replica", str(replica), "--gpu", str(gpu), "--lighthouse", lighthouse, "--steps", str(steps),
         "--exit-at-step", str(exit_at)],
        stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)


def _result(proc, timeout=180):
    out, err = proc.communicate(timeout=timeout)
    lines = [l for l in out.splitlines() if l.startswith("{")]
    assert proc.returncode == 0 and lines, f"rc={proc.returncode}\nstdout={out[-2000:]}\nstderr={err[-3000:]}"
    return json.loads(lines[-1])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_replica_leaves_and_heals_over_nvlink():
    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=200, quorum_tick_ms=20, heartbeat_timeout_ms=1000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    steps = 20
    try:
        p0 = _spawn(0, 0, addr, steps)
        p1 = _spawn(1, 1, addr, steps, exit_at=6)
        assert p1.wait(timeout=120) == 17  # left between steps
        time.sleep(0.5)
        p1b = _spawn(1, 1, addr, steps)  # restarted: new identity, step 0 -> heals from replica 0
        r0, r1 = _result(p0), _result(p1b)
        assert r0["step"] == r1["step"] >= steps
        assert r0["errored"] == "None" and r1["errored"] == "None"
        assert r0["max_participants"] == 2 and r1["max_participants"] == 2
        assert abs(r0["checksum"] - r1["checksum"]) <= 1e-6 * max(1.0, r0["abssum"])
    finally:
        for p in (p0, p1, locals().get("p1b")):
            if p is not None and p.poll() is None:
                p.kill()
        lh.shutdown()
