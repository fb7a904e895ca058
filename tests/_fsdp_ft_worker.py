"""Child of tests/test_fsdp_ft_cpu.py: one rank of one replica group training with stock PyTorch FSDP2
(`fully_shard`) inside the group and a real Manager for the replicate dimension, the way torchtitan uses
the reference (ft_init_device_mesh + fully_shard; torchft/fsdp_test.py:82-92).  Groups start from
different weights: the first quorum (init_sync) equalises them by healing the sharded state dict.
``--exit-at-step N`` makes the group leave between steps."""
import argparse
import json
import os
import sys
import time
from datetime import timedelta

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist
from torch import nn
from torch.distributed import TCPStore
from torch.distributed.fsdp import fully_shard
from torch.distributed.tensor import DTensor

from torchft_b200 import Manager, Optimizer, ProcessGroupGloo
from torchft_b200.checkpointing.http_transport import HTTPTransport
from torchft_b200.device_mesh import ft_init_device_mesh


def local(t: torch.Tensor) -> torch.Tensor:
    return t.to_local() if isinstance(t, DTensor) else t


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--group", type=int, required=True)
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--init-port", type=int, required=True)
    ap.add_argument("--store-port", type=int, required=True)
    ap.add_argument("--lighthouse", required=True)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--exit-at-step", type=int, default=-1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--hold-step", type=int, default=10 ** 9,
                    help="from this step on keep training until a second group has been seen, then stop at a multiple of 5")
    a = ap.parse_args()
    world = 2
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{a.init_port}", rank=a.rank, world_size=world)
    store = TCPStore("127.0.0.1", a.store_port, is_master=(a.rank == 0), wait_for_workers=False)  # noqa: F841 (kept alive)
    timeout = timedelta(seconds=20)

    torch.manual_seed(100 + a.seed)  # same weights on both ranks of a group, different between groups
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 8))
    holder = {}

    def state_dict():
        # healing moves this rank's shards: rank r of the healthy group serves rank r of the joining one
        return {"model": {k: local(v).clone() for k, v in holder["model"].state_dict().items()},
                "optim": {k: {n: local(x).clone() if isinstance(x, torch.Tensor) else x for n, x in st.items()}
                          for k, st in holder["opt"].state_dict()["state"].items()}}

    def load_state_dict(sd):
        with torch.no_grad():
            for k, v in holder["model"].state_dict().items():
                local(v).copy_(sd["model"][k])
            cur = holder["opt"].state_dict()["state"]
            for k, st in sd["optim"].items():
                for n, x in st.items():
                    if isinstance(x, torch.Tensor) and k in cur:
                        local(cur[k][n]).copy_(x)

    manager = Manager(
        pg=ProcessGroupGloo(timeout=timeout), min_replica_size=1, load_state_dict=load_state_dict, state_dict=state_dict,
        replica_id=f"fsdp_{a.group}", store_addr="127.0.0.1", store_port=a.store_port, rank=a.rank, world_size=world,
        lighthouse_addr=a.lighthouse, port=0, hostname="127.0.0.1", timeout=timeout, quorum_timeout=timedelta(seconds=40),
        connect_timeout=timedelta(seconds=20), use_async_quorum=False, checkpoint_transport=HTTPTransport(timeout, num_chunks=0))
    mesh = ft_init_device_mesh(device_type="cpu", mesh_shape=(2, world), mesh_dim_names=("dp_replicate", "dp_shard"),
                               replicate_dim=0, manager=manager)
    for layer in model:
        if isinstance(layer, nn.Linear):
            fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    inner = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    for p in model.parameters():
        # momentum buffers exist from the start (zeros give the same first step), so that a freshly started
        # group has somewhere to receive a healthy group's momentum
        inner.state[p]["momentum_buffer"] = torch.zeros_like(p)
    holder.update(model=model, opt=inner)
    opt = Optimizer(manager, inner)

    rejoined = False
    while True:
        step = manager.current_step()
        if step >= a.steps and (a.hold_step > a.steps or rejoined) and step % 5 == 0:
            break
        if step == a.exit_at_step:
            os._exit(17)
        g = torch.Generator().manual_seed(1000 * a.group + 10 * a.rank + step)
        x, y = torch.randn(8, 16, generator=g), torch.randn(8, 8, generator=g)
        opt.zero_grad()
        (model(x) - y).square().mean().backward()
        opt.step()
        if step >= a.hold_step and not rejoined:
            if manager.num_participants() >= 2:
                rejoined = True
            else:
                time.sleep(0.05)  # alone: do not race ahead of the group that is starting up
    sums = [float(local(p).detach().double().sum()) for p in model.parameters()]
    print(json.dumps({"group": a.group, "rank": a.rank, "step": manager.current_step(), "sums": sums,
                      "participants": manager.num_participants(), "batches": manager.batches_committed()}), flush=True)
    manager.shutdown(wait=False)
    os._exit(0)


if __name__ == "__main__":
    main()
