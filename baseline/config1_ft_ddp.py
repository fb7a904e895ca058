"""FT-DDP plumbing scenario on the unmodified reference (CPU, Gloo): two replica groups of one rank train a
LeNet-style CNN on seeded synthetic images (batch 64, SGD lr 1e-3 momentum 0.9, 100 steps) under the reference's
``Manager``, ``DistributedDataParallel`` and ``OptimizerWrapper`` with ``ProcessGroupGloo`` and the default HTTP
checkpoint transport; replica 1 is killed at step 20 and started again, and heals from its peer.

    python baseline/config1_ft_ddp.py            # launcher; prints one JSON line
    python baseline/config1_ft_ddp.py --impl ours   # the same script on the product package (same public names)

The control plane is the pure-Python stand-in (``torchft_standin.py``): the reference's Rust extension cannot be
built offline.  With ``--impl reference`` (the default) nothing of the product package is imported; ``--impl ours``
runs the very same worker on ``torchft_b200``, whose public names are the reference's.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from datetime import timedelta

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def worker(a) -> int:
    if a.impl == "reference":
        from reference_arm import load_reference

        torchft, _ = load_reference()
    else:  # the same script on the product: the public names are the same
        sys.path.insert(0, os.path.dirname(HERE))
        import torchft_b200 as torchft
    import torch
    from torch import nn, optim
    from torch.distributed import TCPStore

    torch.manual_seed(a.replica + 10 * a.generation)  # different weights: the quorum (init_sync / healing) equalises them
    model = nn.Sequential(nn.Conv2d(3, 6, 5), nn.ReLU(), nn.MaxPool2d(2), nn.Conv2d(6, 16, 5), nn.ReLU(), nn.MaxPool2d(2),
                          nn.Flatten(), nn.Linear(400, 120), nn.ReLU(), nn.Linear(120, 84), nn.ReLU(), nn.Linear(84, 10))
    opt = optim.SGD(model.parameters(), lr=1e-3, momentum=0.9)

    def load_state_dict(sd):
        model.load_state_dict(sd["model"])
        opt.load_state_dict(sd["optim"])

    def state_dict():
        return {"model": model.state_dict(), "optim": opt.state_dict()}

    store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    timeout = timedelta(seconds=20)
    manager = torchft.Manager(
        pg=torchft.ProcessGroupGloo(timeout=timeout), min_replica_size=1, load_state_dict=load_state_dict,
        state_dict=state_dict, replica_id=f"cfg1_{a.replica}", store_addr="127.0.0.1", store_port=store.port, rank=0,
        world_size=1, lighthouse_addr=a.lighthouse, port=0, hostname="127.0.0.1", timeout=timeout,
        quorum_timeout=timedelta(seconds=60), connect_timeout=timedelta(seconds=20), use_async_quorum=False)
    ddp = torchft.DistributedDataParallel(manager, model)
    optimizer = torchft.Optimizer(manager, opt)
    crit = nn.CrossEntropyLoss()
    failed = 0
    while manager.current_step() < a.steps:
        step = manager.current_step()
        if step == a.kill_at and a.generation == 0 and a.replica == 1:
            os._exit(17)  # the failure: this replica is gone
        g = torch.Generator().manual_seed(100000 * a.replica + step)
        x = torch.randn(64, 3, 32, 32, generator=g)
        y = torch.randint(0, 10, (64,), generator=g)
        optimizer.zero_grad()
        crit(ddp(x), y).backward()
        optimizer.step()
        failed += int(manager.current_step() == step)
        if manager.current_step() >= a.hold and manager.num_participants() < 2:
            time.sleep(0.05)  # the survivor paces itself near the end so that the restarted replica can catch up
    checksum = float(sum(p.detach().double().sum().item() for p in model.parameters()))
    print(json.dumps({"replica": a.replica, "step": manager.current_step(), "checksum": checksum, "failed_commits": failed,
                      "participants": manager.num_participants()}), flush=True)
    manager.shutdown(wait=False)
    os._exit(0)


def launcher(a) -> int:
    if a.impl == "reference":
        import torchft_standin as cp
    else:
        sys.path.insert(0, os.path.dirname(HERE))
        from torchft_b200 import _ftcp as cp

    lh = cp.LighthouseServer("[::]:0", 1, join_timeout_ms=200, quorum_tick_ms=20, heartbeat_timeout_ms=1000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]

    def spawn(replica, generation):
        return subprocess.Popen([sys.executable, os.path.abspath(__file__), "--worker", "--replica", str(replica),
                                 "--generation", str(generation), "--lighthouse", addr, "--steps", str(a.steps),
                                 "--kill-at", str(a.kill_at), "--hold", str(a.steps - 30), "--impl", a.impl],
                                stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)

    t0 = time.time()
    p0, p1 = spawn(0, 0), spawn(1, 0)
    procs = [p0, p1]
    try:
        assert p1.wait(timeout=300) == 17
        p1b = spawn(1, 1)
        procs.append(p1b)
        res = []
        for p in (p0, p1b):
            out, err = p.communicate(timeout=600)
            lines = [l for l in out.splitlines() if l.startswith("{")]
            if p.returncode != 0 or not lines:
                raise RuntimeError(f"worker rc={p.returncode}\n{out[-1000:]}\n{err[-3000:]}")
            res.append(json.loads(lines[-1]))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()
    same = abs(res[0]["checksum"] - res[1]["checksum"]) <= 1e-9 * max(1.0, abs(res[0]["checksum"]))
    print(json.dumps({"impl": a.impl, "scenario": "FT-DDP CPU/gloo, 2 groups x 1, LeNet CNN, replica 1 killed at step "
                      f"{a.kill_at} and healed from its peer, {a.steps} steps", "completed": True, "replicas_equal": same,
                      "final_step": [r["step"] for r in res], "survivor_steps_lost": res[0]["failed_commits"],
                      "wall_s": round(time.time() - t0, 1),
                      "control_plane": "pure-Python stand-in for torchft._torchft" if a.impl == "reference" else "C++"}))
    return 0 if same else 1


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--worker", action="store_true")
    ap.add_argument("--impl", default="reference", choices=["reference", "ours"])
    ap.add_argument("--replica", type=int, default=0)
    ap.add_argument("--generation", type=int, default=0)
    ap.add_argument("--lighthouse", default="")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--kill-at", type=int, default=20)
    ap.add_argument("--hold", type=int, default=70)
    args = ap.parse_args()
    sys.exit(worker(args) if args.worker else launcher(args))
