"""torchrun child of tests/test_hsdp_gpu_multi.py: the sharded Llama trainer over 2+ GPUs with
(a) torch.distributed/NCCL collectives, (b) peer-memory kernels, (c) peer-memory kernels with
the reduce-scatter fused into the wgrad GEMM epilogue, (d) as (c) with the all-gather fused into
the forward GEMMs; all must produce the same gradient shards and the same loss trajectory."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from torchft_b200.models.llama import LLAMA_TINY
from torchft_b200.ops import kernels as K
from torchft_b200.parallel.hsdp import ShardedLlamaTrainer
from torchft_b200.parallel.shard_comm import TorchShardComm
from torchft_b200.parallel.team import PeerShardComm


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg, B, S = LLAMA_TINY, 2, 128
    g = torch.Generator().manual_seed(100 + rank)
    tok = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).to(dev)

    def run(comm, fused, fused_ag=False):
        tr = ShardedLlamaTrainer(cfg, B, S, dev, shard_comm=comm, seed=3, logit_chunks=1, fused_reduce_scatter=fused,
                                 fused_all_gather=fused_ag)
        assert tr.fused_rs == fused and tr.fused_ag == fused_ag
        if fused_ag:
            assert tr._ga_units == list(range(1, cfg.n_units))
        losses = []
        for _ in range(3):
            losses.append(tr.train_step(tok[:, :-1], tok[:, 1:]).item())
        torch.cuda.synchronize()
        K.check_status(dev)
        return tr, losses

    ref, ref_losses = run(TorchShardComm(dist.group.WORLD), False)
    out = {"rank": rank, "ref_losses": ref_losses}
    for name, fused, ag in (("peer", False, False), ("fused", True, False), ("fused_ag", True, True)):
        comm = PeerShardComm(dist.group.WORLD, dev, arena_bytes=256 << 20)
        tr, losses = run(comm, fused, ag)
        comm.team.check()
        worst = 0.0
        for u in range(cfg.n_units):
            a, b = tr.g_shard[u].float(), ref.g_shard[u].float()
            worst = max(worst, ((a - b).norm() / (b.norm() + 1e-9)).item())
        out[name] = {"losses": losses, "grad_rel_err": worst}
    print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
