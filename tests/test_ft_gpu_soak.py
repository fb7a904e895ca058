"""Soak of the GPU fault-tolerance path (needs 2 GPUs): one replica keeps training while the other joins, heals
over NVLink peer memory, trains and leaves again a hundred times in a row -- every time as a new replica with
fresh weights, every departure between steps with nothing in flight.  No hang, no failed commit on the
survivor, a hundred heals, and identical weights at the end.  NVLS is off and all kernels use plain peer
loads.  (A replica that dies while one of its kernels is in flight is deliberately not part of any GPU test: the GPUs are shared.)"""
import json
import os
import subprocess
import sys
import time

import pytest
import torch
import torch.distributed as dist

from torchft_b200._ftcp import LighthouseServer

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ft_gpu_soak_worker.py")
CYCLES = int(os.environ.get("FTB200_SOAK_CYCLES", "100"))


def _soak(cycles, cpu, limit_s=420.0):
    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10, heartbeat_timeout_ms=400)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    control = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = []
    try:
        for role, gpu in (("anchor", 0), ("cycler", 1)):
            procs.append(subprocess.Popen(
                [sys.executable, WORKER, "--role", role, "--gpu", str(gpu), "--lighthouse", addr, "--control",
                 f"127.0.0.1:{control.port}", "--cycles", str(cycles)] + (["--cpu"] if cpu else []),
                stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env))
        # wait for both; when one of them ends badly the other is stopped at once instead of running into its own limit
        deadline = time.time() + limit_s
        while any(p.poll() is None for p in procs):
            if any(p.poll() not in (None, 0) for p in procs) or time.time() > deadline:
                break
            time.sleep(0.2)
        outs = []
        for p in procs:
            if p.poll() is None:
                p.kill()
            outs.append(p.communicate())
        results = {}
        for p, (out, err) in zip(procs, outs):
            lines = [l for l in out.splitlines() if l.startswith("{")]
            assert p.returncode == 0 and lines, (
                f"rc={p.returncode}\nstdout={out[-2000:]}\nstderr={err[-3000:]}\n"
                f"other stdout={outs[1 - procs.index(p)][0][-1000:]}\nother stderr={outs[1 - procs.index(p)][1][-2000:]}")
            r = json.loads(lines[-1])
            results[r["role"]] = r
        anchor, cycler = results["anchor"], results["cycler"]
        print("soak:", json.dumps(results))
        assert cycler["heals"] == cycles + 1
        assert anchor["errored"] == "None" and cycler["errored"] == "None"
        assert anchor["commit_failures"] == 0, anchor
        assert anchor["step"] == cycler["step"]
        assert abs(anchor["checksum"] - cycler["checksum"]) <= 1e-6 * max(1.0, anchor["abssum"])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_hundred_leave_and_heal_cycles():
    _soak(CYCLES, cpu=False)


def test_leave_and_heal_cycles_on_cpu():
    """The same scenario over Gloo and the HTTP transport: the host-side logic of the soak, without GPUs."""
    _soak(8, cpu=True)
