"""Child process of tests/test_ft_gpu_soak.py: one replica group on one GPU, FT-DDP over ProcessGroupB200.

``--role anchor`` trains without interruption.  ``--role cycler`` joins, is healed over NVLink, trains a few
steps, and leaves again, ``--cycles`` times: every cycle it comes back as a new replica (new manager, new
identity, freshly randomised weights and optimizer), exactly as a restarted process would, and it leaves only
between steps, after a device synchronisation, with nothing of its own in flight.  The survivor learns of every
departure on the host (heartbeat expiry, then a quorum without the leaver) before its next launch.  After the
last cycle the two agree through the control store on a step at which both stop and print a checksum."""
import argparse
import json
import os
import sys
import time
from datetime import timedelta

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
from torch import nn, optim
from torch.distributed import TCPStore

from torchft_b200 import DistributedDataParallel, Manager, Optimizer
from torchft_b200.checkpointing.p2p_transport import P2PTransport
from torchft_b200.parallel.team import ProcessGroupB200


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", choices=["anchor", "cycler"], required=True)
    ap.add_argument("--gpu", type=int, required=True)
    ap.add_argument("--lighthouse", required=True)
    ap.add_argument("--control", required=True, help="host:port of the test's control store")
    ap.add_argument("--cycles", type=int, default=100)
    ap.add_argument("--steps-per-cycle", type=int, default=3)
    ap.add_argument("--cpu", action="store_true", help="same scenario on CPU over Gloo and the HTTP transport (logic check)")
    a = ap.parse_args()
    if a.cpu:
        dev = torch.device("cpu")
    else:
        torch.cuda.set_device(a.gpu)
        dev = torch.device("cuda", a.gpu)
    host, port = a.control.rsplit(":", 1)
    control = TCPStore(host, int(port), is_master=False, wait_for_workers=False)
    model = nn.Sequential(nn.Linear(64, 256), nn.ReLU(), nn.Linear(256, 16)).to(dev)
    crit = nn.MSELoss()
    store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    timeout = timedelta(seconds=5)
    if a.cpu:
        from torchft_b200.process_group import ProcessGroupGloo

        pg = ProcessGroupGloo(timeout=timeout)
    else:
        pg = ProcessGroupB200(timeout=timeout, arena_bytes=8 << 20, staging_bytes=8 << 20, device=dev)

    def sync():
        if not a.cpu:
            torch.cuda.synchronize()

    def transport():
        if a.cpu:
            from torchft_b200.checkpointing.http_transport import HTTPTransport

            return HTTPTransport(timeout=timeout, num_chunks=0)
        return P2PTransport(timeout=timeout, device=dev, state_dict=None)

    stats = {"commit_failures": 0, "steps": 0, "joint_steps": 0, "heals": 0}

    def fresh(seed):
        torch.manual_seed(seed)
        for m in model:
            if hasattr(m, "reset_parameters"):
                m.reset_parameters()
        opt = optim.SGD(model.parameters(), lr=0.05, momentum=0.9)

        def load_state_dict(sd):
            model.load_state_dict(sd["model"])
            opt.load_state_dict(sd["optim"])

        def state_dict():
            return {"model": model.state_dict(), "optim": opt.state_dict()}

        manager = Manager(
            pg=pg, min_replica_size=1, load_state_dict=load_state_dict, state_dict=state_dict,
            replica_id=f"soak_{a.role}", store_addr="127.0.0.1", store_port=store.port, rank=0, world_size=1,
            lighthouse_addr=a.lighthouse, port=0, hostname="127.0.0.1", timeout=timeout,
            quorum_timeout=timedelta(seconds=20), connect_timeout=timedelta(seconds=10),
            checkpoint_transport=transport(), use_async_quorum=False)
        return manager, DistributedDataParallel(manager, model), Optimizer(manager, opt)

    def one_step(manager, ddp, optimizer):
        optimizer.zero_grad()  # synchronous quorum: a joiner is healed (and its step set) in here
        step = manager.current_step()
        n = manager.num_participants()
        g = torch.Generator().manual_seed(7919 * step + (0 if a.role == "anchor" else 1))
        x = torch.randn(32, 64, generator=g).to(dev)
        y = torch.randn(32, 16, generator=g).to(dev)
        crit(ddp(x), y).backward()
        optimizer.step()
        stats["steps"] += 1
        stats["joint_steps"] += int(n >= 2)
        if manager.current_step() == step:
            stats["commit_failures"] += 1
        return n

    def finish(manager):
        sync()
        checksum = float(sum(p.detach().double().sum().item() for p in model.parameters()))
        absum = float(sum(p.detach().double().abs().sum().item() for p in model.parameters()))
        print(json.dumps({"role": a.role, "step": manager.current_step(), "checksum": checksum, "abssum": absum,
                          "errored": str(pg.errored()), **stats}), flush=True)
        manager.shutdown(wait=False)
        os._exit(0)

    t_start = time.time()
    if a.role == "anchor":
        manager, ddp, optimizer = fresh(0)
        target = None
        while True:
            if target is None and control.check(["target"]):
                target = int(control.get("target"))
            if target is not None and manager.current_step() >= target:
                finish(manager)
            n = one_step(manager, ddp, optimizer)
            if manager.current_step() == 3:
                control.set("anchor_ready", "1")  # the cycler's first join must find a running job
            if n < 2:
                time.sleep(0.01)  # alone: keep asking for quorums (that is how a joiner gets in) without racing ahead
            if time.time() - t_start > 400:
                print(json.dumps({"role": a.role, "error": "no target after 400 s", **stats}), flush=True)
                os._exit(3)
    else:
        control.wait(["anchor_ready"], timedelta(seconds=120))
        for cycle in range(a.cycles + 1):
            manager, ddp, optimizer = fresh(1000 + cycle)
            before = float(sum(p.detach().double().sum().item() for p in model.parameters()))
            n = one_step(manager, ddp, optimizer)  # heals in here
            after = float(sum(p.detach().double().sum().item() for p in model.parameters()))
            if n < 2 or after == before:
                print(json.dumps({"role": a.role, "error": f"cycle {cycle}: not healed into a quorum of two "
                                                           f"(participants {n}, step {manager.current_step()})", **stats}), flush=True)
                os._exit(4)
            stats["heals"] += 1
            if cycle % 10 == 0:
                print(f"[cycler] cycle {cycle} healed at step {manager.current_step()} after {time.time() - t_start:.1f} s",
                      file=sys.stderr, flush=True)
            if cycle == a.cycles:
                # the last join stays: agree on a final step
                target = manager.current_step() + 20
                control.set("target", str(target))
                while manager.current_step() < target:
                    one_step(manager, ddp, optimizer)
                finish(manager)
            for _ in range(a.steps_per_cycle - 1):
                one_step(manager, ddp, optimizer)
            sync()  # leave between steps: nothing of ours is in flight
            manager.shutdown(wait=False)
            del manager, ddp, optimizer


if __name__ == "__main__":
    main()
