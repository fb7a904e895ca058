"""ProcessGroupB200 across real GPUs (needs >= 2): every collective of the c10d surface checked numerically
at ragged, small and window-exceeding sizes, point-to-point transfers, the quantised allreduce helper and
the process-group checkpoint transport on top of it.  One process per GPU, plain peer loads (no NVLS)."""
import json
import os
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu
WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_pg_b200_worker.py")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("world", [2, 4])
def test_collectives_across_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    store = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, WORKER, "--rank", str(r), "--world", str(world), "--store",
                               f"127.0.0.1:{store.port}"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
             for r in range(world)]
    try:
        for p in procs:
            out, err = p.communicate(timeout=240)
            lines = [l for l in out.splitlines() if l.startswith("{")]
            assert p.returncode == 0 and lines, f"rc={p.returncode}\nstdout={out[-2000:]}\nstderr={err[-3000:]}"
            res = json.loads(lines[-1])
            bad = [k for k, v in res["checks"].items() if not v]
            assert not bad and res["errored"] == "None", (res["rank"], bad, res["errored"])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
