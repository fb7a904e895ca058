#!/usr/bin/env python
"""Fault-tolerant HSDP training of a Llama-3 style decoder on one multi-GPU box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 train_hsdp.py --model llama3-8b --seq-len 8192 --steps 100 --replica-groups 2

GPUs are split into ``--replica-groups`` groups; inside a group parameters, gradients and
AdamW state are sharded (FSDP style, NVLink peer-memory all-gather / reduce-scatter),
across groups gradients are averaged through the fault-tolerant Manager.  A group that
disappears (``--kill-group G --kill-step S`` makes group G exit at step S to demonstrate)
is dropped from the quorum within the heartbeat timeout and the others continue; relaunch
its ranks and they heal from a surviving group over NVLink.  ``--ckpt-dir D --ckpt-every N`` writes
a durable checkpoint every N committed steps (replica group 0 only: the groups hold identical
state) and resumes from the newest complete one when the whole job is started again.
The reference reaches the same layout through torchtitan + torchft; here the trainer is
part of the framework (:mod:`torchft_b200.parallel.hsdp`).  Without a GPU the same script runs on CPU
over Gloo (use ``--model llama-tiny --seq-len 16``), which is how the test suite exercises it.
"""

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from torchft_b200.bench_support import make_ft_manager
from torchft_b200.models.llama import CONFIGS
from torchft_b200.ops import kernels as K
from torchft_b200.parallel.hsdp import ShardedLlamaTrainer
from torchft_b200.parallel.shard_comm import LocalShardComm


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-1b", choices=sorted(CONFIGS))
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--replica-groups", type=int, default=2)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--kill-group", type=int, default=-1)
    ap.add_argument("--kill-step", type=int, default=-1)
    ap.add_argument("--ckpt-dir", default="")
    ap.add_argument("--ckpt-every", type=int, default=0)
    a = ap.parse_args()

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")  # CPU: Gloo everywhere, for trying things out
    cfg = CONFIGS[a.model]
    n_groups = min(a.replica_groups, world)
    shard = world // n_groups
    group_id, group_rank = rank // shard, rank % shard
    shard_comm = LocalShardComm()
    if world > 1:
        if use_cuda:
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
        groups = [dist.new_group(list(range(g * shard, (g + 1) * shard))) for g in range(n_groups)]
        if shard > 1 and use_cuda:
            from torchft_b200.parallel.team import PeerShardComm

            pbytes = sum(cfg.unit_numel(u) for u in range(cfg.n_units)) * 2
            shard_comm = PeerShardComm(groups[group_id], dev, arena_bytes=pbytes // shard + (5 << 30))
        elif shard > 1:
            from torchft_b200.parallel.shard_comm import TorchShardComm

            shard_comm = TorchShardComm(groups[group_id])
    grad_bytes = sum(cfg.unit_numel(u) for u in range(cfg.n_units)) * 2 // shard
    lighthouse, manager = make_ft_manager(rank, world, n_groups, shard, group_id, group_rank, dev,
                                          arena_bytes=grad_bytes + (64 << 20), min_replica_size=1)
    trainer = ShardedLlamaTrainer(cfg, a.micro_batch, a.seq_len, dev, shard_comm=shard_comm, manager=manager, lr=a.lr,
                                  replica_alloc=manager._pg.alloc if n_groups > 1 and use_cuda else None)
    manager.register_state_dict_fn("trainer", trainer.load_state_dict, trainer.state_dict)

    g = torch.Generator().manual_seed(1234 + rank)
    ckpt = None
    if a.ckpt_dir:
        from torchft_b200.checkpointing.durable import DurableCheckpointer

        ckpt = DurableCheckpointer(manager, a.ckpt_dir, rank=group_rank, world_size=shard, every=a.ckpt_every)
        extra = ckpt.load_latest()
        if extra is not None:
            g.set_state(extra["data_rng"])
            print(f"[rank {rank}] resumed from step {manager.current_step()}", flush=True)
    t0 = time.time()
    while manager.current_step() < a.steps:
        step = manager.current_step()
        if group_id == a.kill_group and step == a.kill_step:
            print(f"[rank {rank}] group {group_id} leaves at step {step}", flush=True)
            os._exit(1)
        tok = torch.randint(0, cfg.vocab_size, (a.micro_batch, a.seq_len + 1), generator=g).to(dev)
        loss = trainer.train_step(tok[:, :-1], tok[:, 1:])
        if ckpt is not None and group_id == 0:
            ckpt.maybe_save(extra={"data_rng": g.get_state()})
        if rank == 0 and step % 5 == 0:
            print(f"step {step} loss {loss.item():.4f} participants {manager.num_participants()} "
                  f"{(time.time() - t0):.1f}s", flush=True)
    if use_cuda:
        K.check_status(dev)
    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()


if __name__ == "__main__":
    main()
