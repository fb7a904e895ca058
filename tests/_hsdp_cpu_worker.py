"""Child of tests/test_llama_engine.py::test_sharded_trainer_two_gloo_ranks: one rank of a two-rank
shard group on CPU.  Rank r runs forward/backward on its own micro-batch, saves the gathered
gradient of every unit (rank 0), then trains a few steps and prints its losses."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from torchft_b200.models.llama import LLAMA_TINY
from torchft_b200.parallel.hsdp import ShardedLlamaTrainer
from torchft_b200.parallel.shard_comm import TorchShardComm


def main() -> None:
    rank, world, port, out_path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    cfg, B, S = LLAMA_TINY, 1, 16
    g = torch.Generator().manual_seed(7)
    tok = torch.randint(0, cfg.vocab_size, (world * B, S + 1), generator=g)  # the job's batch; rank r takes row r
    tr = ShardedLlamaTrainer(cfg, B, S, torch.device("cpu"), shard_comm=TorchShardComm(dist.group.WORLD), seed=3, lr=1e-2,
                             max_grad_norm=1e9)
    mine = tok[rank * B : (rank + 1) * B]
    first_loss = float(tr.forward_backward(mine[:, :-1], mine[:, 1:]))
    tr._finish_comm()
    grads = []
    for u in range(cfg.n_units):
        full = [torch.empty_like(tr.g_shard[u]) for _ in range(world)]
        dist.all_gather(full, tr.g_shard[u])
        grads.append(torch.cat(full)[: cfg.unit_numel(u)].float())
    if rank == 0:
        torch.save(grads, out_path)
    tr.optimizer_step()
    losses = [first_loss] + [float(tr.train_step(mine[:, :-1], mine[:, 1:])) for _ in range(3)]
    print(json.dumps({"rank": rank, "losses": losses}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
