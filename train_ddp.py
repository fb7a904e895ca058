#!/usr/bin/env python
"""Fault-tolerant DDP example: a LeNet-style CNN on synthetic 3x32x32 images.

Start a lighthouse, then one process (group) per replica:

    python -m torchft_b200.lighthouse_cli --min_replicas 1 --join_timeout_ms 1000 &
    TORCHFT_LIGHTHOUSE=http://localhost:29510 REPLICA_GROUP_ID=0 NUM_REPLICA_GROUPS=2 \
        torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 1 --master-port 29600 train_ddp.py
    TORCHFT_LIGHTHOUSE=http://localhost:29510 REPLICA_GROUP_ID=1 NUM_REPLICA_GROUPS=2 \
        torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 1 --master-port 29601 train_ddp.py

Kill either trainer and restart it: it rejoins the quorum, copies the weights from the
surviving replica and continues; the survivor never stops.  ``USE_PEER=1`` on GPUs of one
NVSwitch domain selects the NVLink peer-memory process group and state transfer; ``USE_NCCL=0``
selects Gloo for the replica dimension on GPUs (the default is NCCL on GPUs, Gloo on CPU).
Counterpart of the reference's train_ddp.py (CIFAR-10 replaced by seeded synthetic data).
"""

import logging
import os
import sys
from datetime import timedelta

import torch
from torch import nn, optim

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from torchft_b200 import DistributedDataParallel, DistributedSampler, Manager, Optimizer, ProcessGroupGloo, ProcessGroupNCCL
from torchft_b200.checkpointing.pg_transport import PGTransport
from torchft_b200.launch.runner import install_fault_handlers
from torchft_b200.models.lenet import LeNet

logging.basicConfig(level=logging.INFO)


class SyntheticImages(torch.utils.data.Dataset):
    def __init__(self, n: int = 8192, seed: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        self.x = torch.randn(n, 3, 32, 32, generator=g)
        self.y = torch.randint(0, 10, (n,), generator=g)

    def __len__(self) -> int:
        return len(self.x)

    def __getitem__(self, i):
        return self.x[i], self.y[i]


def main() -> None:
    replica_group = int(os.environ.get("REPLICA_GROUP_ID", 0))
    num_groups = int(os.environ.get("NUM_REPLICA_GROUPS", 2))
    steps = int(os.environ.get("STEPS", 100))
    use_cuda = torch.cuda.is_available()
    # GPU_OFFSET: first GPU of this replica group when several groups share one box (torchrun numbers
    # LOCAL_RANK from 0 in every group)
    gpu = int(os.environ.get("LOCAL_RANK", 0)) + int(os.environ.get("GPU_OFFSET", 0))
    device = torch.device("cuda", gpu) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)

    data = SyntheticImages()
    sampler = DistributedSampler(data, replica_rank=replica_group, num_replica_groups=num_groups, group_rank=0,
                                 num_replicas=1, shuffle=True)
    loader = torch.utils.data.DataLoader(data, batch_size=64, sampler=sampler, num_workers=0)

    model = LeNet().to(device)
    opt = optim.SGD(model.parameters(), lr=1e-3, momentum=0.9)

    def load_state_dict(sd):
        model.load_state_dict(sd["model"])
        opt.load_state_dict(sd["optim"])

    def state_dict():
        return {"model": model.state_dict(), "optim": opt.state_dict()}

    timeout = timedelta(seconds=30)
    # Replica dimension on GPUs: NVLink peer memory (ProcessGroupB200) unless told otherwise.  It needs all
    # replica groups on one NVSwitch box; USE_PEER=0 (or an explicit USE_NCCL=1) selects NCCL, USE_NCCL=0 Gloo.
    nccl_env = os.environ.get("USE_NCCL")
    use_peer = use_cuda and nccl_env is None and os.environ.get("USE_PEER", "1") == "1"
    if use_peer:
        from torchft_b200.checkpointing.p2p_transport import P2PTransport
        from torchft_b200.parallel.team import ProcessGroupB200

        pg = ProcessGroupB200(timeout=timeout, device=device)
        transport = P2PTransport(timeout=timeout, device=device, state_dict=state_dict)
    else:
        # USE_NCCL=0 keeps the tensors on the GPU but moves the replica dimension to Gloo
        use_nccl = use_cuda and (nccl_env or "1").lower() not in ("0", "false")
        pg = ProcessGroupNCCL(timeout=timeout) if use_nccl else ProcessGroupGloo(timeout=timeout)
        transport = PGTransport(pg, timeout=timeout, device=device)

    manager = Manager(
        pg=pg,
        min_replica_size=1,
        load_state_dict=load_state_dict,
        state_dict=state_dict,
        replica_id=f"train_ddp_{replica_group}",
        timeout=timeout,
        checkpoint_transport=transport,
    )
    install_fault_handlers(manager)  # lets the punisher inject a communication failure (SIGUSR1)
    ddp = DistributedDataParallel(manager, model)
    optimizer = Optimizer(manager, opt)
    criterion = nn.CrossEntropyLoss()

    # PROFILE_DIR=<dir>: trace a few steps with torch.profiler (the manager's record_function scopes such as
    # torchft::manager::allreduce and ::should_commit show up in it) and write chrome traces there
    prof = None
    if os.environ.get("PROFILE_DIR"):
        acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if use_cuda else [])
        prof = torch.profiler.profile(
            activities=acts, schedule=torch.profiler.schedule(wait=5, warmup=2, active=6, repeat=1),
            on_trace_ready=torch.profiler.tensorboard_trace_handler(os.path.join(os.environ["PROFILE_DIR"], f"group{replica_group}")))
        prof.start()

    import time

    t_mark = None  # (time, step) once the first ten steps (quorum set-up, warm-up) are behind us
    while manager.current_step() < steps:
        sampler.set_epoch(manager.current_step())
        for x, y in loader:
            x, y = x.to(device), y.to(device)
            optimizer.zero_grad()          # joins the quorum
            loss = criterion(ddp(x), y)
            loss.backward()                # bucketed gradients are averaged through the manager
            optimizer.step()               # applied only if the step commits
            if manager.current_step() % 10 == 0:
                print(f"[{replica_group}] step={manager.current_step()} batches={manager.batches_committed()} "
                      f"participants={manager.num_participants()} loss={loss.item():.4f}", flush=True)
            if prof is not None:
                prof.step()
            if t_mark is None and manager.current_step() >= 10:
                if use_cuda:
                    torch.cuda.synchronize()
                t_mark = (time.perf_counter(), manager.current_step())
            # a durable checkpoint would save state_dict(), manager.state_dict() and the loader position here
            if manager.current_step() >= steps:
                break
    if prof is not None:
        prof.stop()
    if t_mark is not None and manager.current_step() > t_mark[1]:
        if use_cuda:
            torch.cuda.synchronize()
        n = manager.current_step() - t_mark[1]
        print(f"[{replica_group}] {n} committed steps in {time.perf_counter() - t_mark[0]:.3f} s "
              f"({(time.perf_counter() - t_mark[0]) / n * 1e3:.3f} ms/step, replica dimension: {type(pg).__name__})", flush=True)
    manager.shutdown()


if __name__ == "__main__":
    main()
