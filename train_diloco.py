#!/usr/bin/env python
"""(Streaming) DiLoCo example: an MLP split into fragments, AdamW inside, Nesterov SGD outside.

    python -m torchft_b200.lighthouse_cli --min_replicas 1 --join_timeout_ms 1000 &
    TORCHFT_LIGHTHOUSE=http://localhost:29510 REPLICA_GROUP_ID=0 NUM_REPLICA_GROUPS=2 USE_STREAMING=1 \
        torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 1 --master-port 29600 train_diloco.py

Each replica takes ``sync_every`` local steps between synchronisations; with
``USE_STREAMING=1`` the model is cut into two fragments that synchronise alternately and
whose allreduce starts ``fragment_sync_delay`` steps early.  ``QUANTIZE=1`` sends the
pseudo-gradients as block-scaled fp8.  Counterpart of the reference's train_diloco.py.
"""

import logging
import os
import sys
from datetime import timedelta

import torch
from torch import nn, optim

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from torchft_b200 import Manager, ProcessGroupGloo, ProcessGroupNCCL
from torchft_b200.checkpointing.http_transport import HTTPTransport
from torchft_b200.local_sgd import DiLoCo

logging.basicConfig(level=logging.INFO)


def build_model(hidden: int = 256, layers: int = 4) -> nn.Sequential:
    blocks = [nn.Sequential(nn.Linear(3 * 32 * 32 if i == 0 else hidden, hidden), nn.ReLU()) for i in range(layers)]
    blocks.append(nn.Sequential(nn.Linear(hidden, 10)))
    return nn.Sequential(*blocks)


def main() -> None:
    replica_group = int(os.environ.get("REPLICA_GROUP_ID", 0))
    steps = int(os.environ.get("STEPS", 200))
    streaming = os.environ.get("USE_STREAMING", "0") == "1"
    quantize = os.environ.get("QUANTIZE", "0") == "1"
    use_cuda = torch.cuda.is_available()
    # GPU_OFFSET: first GPU of this replica group when several groups share one box (torchrun numbers
    # LOCAL_RANK from 0 in every group)
    gpu = int(os.environ.get("LOCAL_RANK", 0)) + int(os.environ.get("GPU_OFFSET", 0))
    device = torch.device("cuda", gpu) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)

    torch.manual_seed(0)  # identical initial weights on every replica
    model = build_model().to(device)
    if streaming:
        half = len(model) // 2
        fragments = [model[:half], model[half:]]
    else:
        fragments = [model]

    inner = optim.AdamW(model.parameters(), lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95))
    outers = [optim.SGD(f.parameters(), lr=0.7, momentum=0.9, nesterov=True) for f in fragments]

    def load_state_dict(sd):
        model.load_state_dict(sd["model"])
        inner.load_state_dict(sd["inner_optim"])

    def state_dict():
        return {"model": model.state_dict(), "inner_optim": inner.state_dict()}

    timeout = timedelta(seconds=30)
    # Replica dimension on GPUs: NVLink peer memory (ProcessGroupB200) unless told otherwise.  It needs all
    # replica groups on one NVSwitch box; USE_PEER=0 (or an explicit USE_NCCL=1) selects NCCL, USE_NCCL=0 Gloo.
    nccl_env = os.environ.get("USE_NCCL")
    use_peer = use_cuda and nccl_env is None and os.environ.get("USE_PEER", "1") == "1"
    if use_peer:
        from torchft_b200.parallel.team import ProcessGroupB200

        pg = ProcessGroupB200(timeout=timeout, device=device)
    else:
        # USE_NCCL=0 keeps the tensors on the GPU but moves the replica dimension to Gloo
        use_nccl = use_cuda and (nccl_env or "1").lower() not in ("0", "false")
        pg = ProcessGroupNCCL(timeout=timeout) if use_nccl else ProcessGroupGloo(timeout=timeout)
    manager = Manager(
        pg=pg,
        min_replica_size=1,
        load_state_dict=load_state_dict,
        state_dict=state_dict,
        replica_id=f"train_diloco_{replica_group}",
        timeout=timeout,
        use_async_quorum=False,  # DiLoCo heals synchronously, before the pseudo-gradient is formed
        checkpoint_transport=HTTPTransport(timeout=timeout, num_chunks=0),
    )
    criterion = nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(1000 + replica_group)
    # RUN=<name>: TensorBoard scalars (loss, committed outer steps, participants) under runs/<name>_group<g>
    writer = None
    if os.environ.get("RUN"):
        from torch.utils.tensorboard import SummaryWriter

        writer = SummaryWriter(os.path.join("runs", f"{os.environ['RUN']}_group{replica_group}"))
    with DiLoCo(manager, fragments, inner, outers, sync_every=20 if streaming else 20,
                fragment_sync_delay=5 if streaming else 0, should_quantize=quantize,
                backup_device=device if use_cuda else None) as diloco:
        import time

        t_mark = None
        for step in range(steps):
            if step == 40:  # two rounds of synchronisations are behind us
                if use_cuda:
                    torch.cuda.synchronize()
                t_mark = time.perf_counter()
            x = torch.randn(64, 3 * 32 * 32, generator=g).to(device)
            y = torch.randint(0, 10, (64,), generator=g).to(device)
            inner.zero_grad()
            loss = criterion(model(x), y)
            loss.backward()
            inner.step()  # DiLoCo's hooks run the quorum / allreduce / outer step when due
            if writer is not None:
                writer.add_scalar("loss", loss.item(), step)
                writer.add_scalar("manager_step", manager.current_step(), step)
            if step % 20 == 0:
                print(f"[{replica_group}] local_step={step} manager_step={manager.current_step()} loss={loss.item():.4f}",
                      flush=True)
        if t_mark is not None and steps > 40:
            if use_cuda:
                torch.cuda.synchronize()
            dt = time.perf_counter() - t_mark
            print(f"[{replica_group}] {steps - 40} inner steps in {dt:.3f} s ({dt / (steps - 40) * 1e3:.3f} ms/step, "
                  f"manager_step={manager.current_step()}, replica dimension: {type(pg).__name__})", flush=True)
    if writer is not None:
        writer.close()
    manager.shutdown()


if __name__ == "__main__":
    main()
