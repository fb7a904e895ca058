"""Child process of tests/test_ft_gpu_multi.py: one replica group on one GPU.

Trains a small MLP with FT-DDP over ProcessGroupB200 (NVLink peer memory) and P2PTransport.
``--exit-at-step N`` makes the process leave *between* steps (after the commit of step N-1,
with no kernel or collective in flight); the parent then restarts it and it heals from the
surviving replica.  Prints one JSON line with a checksum of the final weights."""
import argparse
import json
import os
import sys
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
    ap.add_argument("--replica", type=int, required=True)
    ap.add_argument("--gpu", type=int, required=True)
    ap.add_argument("--lighthouse", required=True)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--exit-at-step", type=int, default=-1)
    ap.add_argument("--hold-step", type=int, default=10, help="from this step on, step slowly until a peer is present")
    a = ap.parse_args()
    torch.cuda.set_device(a.gpu)
    dev = torch.device("cuda", a.gpu)
    torch.manual_seed(a.replica)  # different init: the first quorum must equalise it (init_sync)
    model = nn.Sequential(nn.Linear(64, 256), nn.ReLU(), nn.Linear(256, 16)).to(dev)
    opt = optim.SGD(model.parameters(), lr=0.05, momentum=0.9)

    def load_state_dict(sd):
        model.load_state_dict(sd["model"])
        opt.load_state_dict(sd["optim"])

    def state_dict():
        return {"model": model.state_dict(), "optim": opt.state_dict()}

    store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    timeout = timedelta(seconds=5)
    pg = ProcessGroupB200(timeout=timeout, arena_bytes=8 << 20, staging_bytes=8 << 20, device=dev)
    manager = Manager(
        pg=pg, min_replica_size=1, load_state_dict=load_state_dict, state_dict=state_dict, replica_id=f"gpu_rep{a.replica}",
        store_addr="127.0.0.1", store_port=store.port, rank=0, world_size=1, lighthouse_addr=a.lighthouse, port=0,
        hostname="127.0.0.1", timeout=timeout, quorum_timeout=timedelta(seconds=20), connect_timeout=timedelta(seconds=10),
        checkpoint_transport=P2PTransport(timeout=timeout, device=dev, state_dict=None),
        use_async_quorum=False,  # a joiner heals inside start_quorum, so both sides see the same membership per step
    )
    ddp = DistributedDataParallel(manager, model)
    optimizer = Optimizer(manager, opt)
    crit = nn.MSELoss()
    import time

    max_participants = 0
    rejoined_at = None  # first step >= hold-step that ran with two participants (same on both replicas)
    t_hold = time.time()
    while True:
        step = manager.current_step()
        if rejoined_at is not None and step >= max(a.steps, rejoined_at + 5) and step % 10 == 0:
            break
        if step == a.exit_at_step:
            torch.cuda.synchronize()
            os._exit(17)  # leaves between steps: nothing of ours is in flight
        optimizer.zero_grad()  # synchronous quorum: a joiner is healed (and its step set) in here
        step = manager.current_step()
        n = manager.num_participants()
        g = torch.Generator().manual_seed(1000 * a.replica + step)
        x = torch.randn(32, 64, generator=g).to(dev)
        y = torch.randn(32, 16, generator=g).to(dev)
        crit(ddp(x), y).backward()
        optimizer.step()
        max_participants = max(max_participants, n)
        if step >= a.hold_step and rejoined_at is None:
            if n >= 2:
                rejoined_at = step
            else:
                time.sleep(0.1)  # keep asking for quorums (that is how a joiner gets in) without racing ahead
                if time.time() - t_hold > 150:
                    print(json.dumps({"replica": a.replica, "error": "peer never rejoined"}), flush=True)
                    os._exit(3)
    torch.cuda.synchronize()
    checksum = float(sum(p.detach().double().sum().item() for p in model.parameters()))
    absum = float(sum(p.detach().double().abs().sum().item() for p in model.parameters()))
    print(json.dumps({"replica": a.replica, "step": manager.current_step(), "checksum": checksum, "abssum": absum,
                      "errored": str(pg.errored()), "max_participants": max_participants}), flush=True)
    manager.shutdown(wait=False)
    os._exit(0)


if __name__ == "__main__":
    main()
