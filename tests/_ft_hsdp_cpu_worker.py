"""Child of tests/test_ft_hsdp_cpu.py: one rank of one replica group.  A replica group is a
two-rank gloo job of its own (parameters, gradients and optimizer state sharded between the two
ranks); the groups average their gradient shards through per-rank Managers over ProcessGroupGloo.
``--exit-at-step N`` makes both ranks of the group leave between two steps; the parent starts the
group again with different initial weights and it heals from the surviving group."""
import argparse
import json
import os
import sys
import time
from datetime import timedelta

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist
from torch.distributed import TCPStore

from torchft_b200 import Manager, ProcessGroupGloo
from torchft_b200.models.llama import LLAMA_TINY
from torchft_b200.parallel.hsdp import ShardedLlamaTrainer
from torchft_b200.parallel.shard_comm import TorchShardComm


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--group", type=int, required=True)
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--init-port", type=int, required=True)   # the group's gloo rendezvous
    ap.add_argument("--store-port", type=int, required=True)  # the group's manager store
    ap.add_argument("--lighthouse", required=True)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--exit-at-step", type=int, default=-1)
    ap.add_argument("--hold-step", type=int, default=10 ** 9)
    ap.add_argument("--seed", type=int, default=3)
    ap.add_argument("--async-quorum", type=int, default=0)
    ap.add_argument("--diloco", type=int, default=0, help="streaming DiLoCo over the engine: number of fragments")
    a = ap.parse_args()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{a.init_port}", rank=a.rank, world_size=2)
    store = TCPStore("127.0.0.1", a.store_port, is_master=(a.rank == 0), wait_for_workers=False)
    timeout = timedelta(seconds=20)
    pg = ProcessGroupGloo(timeout=timeout)
    manager = Manager(
        pg=pg, min_replica_size=1, load_state_dict=None, state_dict=None, replica_id=f"hsdp_cpu_{a.group}",
        store_addr="127.0.0.1", store_port=a.store_port, rank=a.rank, world_size=2, lighthouse_addr=a.lighthouse, port=0,
        hostname="127.0.0.1", timeout=timeout, quorum_timeout=timedelta(seconds=40), connect_timeout=timedelta(seconds=20),
        use_async_quorum=bool(a.async_quorum), init_sync=False)
    cfg, B, S = LLAMA_TINY, 1, 16
    tr = ShardedLlamaTrainer(cfg, B, S, torch.device("cpu"), shard_comm=TorchShardComm(dist.group.WORLD),
                             manager=None if a.diloco else manager, seed=a.seed, lr=1e-2)
    manager.register_state_dict_fn("trainer", tr.load_state_dict, tr.state_dict)
    if a.diloco:
        from torchft_b200.parallel.diloco import EngineDiLoCo

        d = EngineDiLoCo(tr, manager, n_fragments=a.diloco, sync_every=2 * a.diloco, fragment_sync_delay=1,
                         fragment_update_alpha=0.5)
        it = 0
        while manager.current_step() < a.steps:
            g = torch.Generator().manual_seed(10000 * a.group + 100 * a.rank + it)
            tok = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g)
            d.train_step(tok[:, :-1], tok[:, 1:])
            it += 1
        sums = []
        for f in d.fragments:  # the global (backup) weights are what the groups must agree on
            for b in f.backup:
                full = [torch.empty_like(b) for _ in range(2)]
                dist.all_gather(full, b)
                sums.append(float(torch.cat(full).double().sum()))
        print(json.dumps({"group": a.group, "rank": a.rank, "step": manager.current_step(), "unit_sums": sums,
                          "max_participants": manager.num_participants(), "errored": str(pg.errored()),
                          "commits": d.commits}), flush=True)
        manager.shutdown(wait=False)
        os._exit(0)

    max_participants, rejoined_at, t_hold = 0, None, time.time()
    while True:
        step = manager.current_step()
        if step >= a.steps and (a.hold_step > a.steps or rejoined_at is not None) and step % 5 == 0:
            break
        if step == a.exit_at_step:
            os._exit(17)  # between steps: nothing in flight
        g = torch.Generator().manual_seed(10000 * a.group + 100 * a.rank + step)
        tok = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g)
        tr.train_step(tok[:, :-1], tok[:, 1:])
        n = manager.num_participants()
        max_participants = max(max_participants, n)
        if step >= a.hold_step and rejoined_at is None:
            if n >= 2:
                rejoined_at = step
            else:
                time.sleep(0.1)
                if time.time() - t_hold > 120:
                    print(json.dumps({"error": "peer never rejoined"}), flush=True)
                    os._exit(3)
    sums = []
    for u in range(cfg.n_units):
        full = [torch.empty_like(tr.master[u]) for _ in range(2)]
        dist.all_gather(full, tr.master[u])
        sums.append(float(torch.cat(full)[: cfg.unit_numel(u)].double().sum()))
    print(json.dumps({"group": a.group, "rank": a.rank, "step": manager.current_step(), "unit_sums": sums,
                      "max_participants": max_participants, "errored": str(pg.errored())}), flush=True)
    manager.shutdown(wait=False)
    os._exit(0)


if __name__ == "__main__":
    main()
