"""Child of tests/test_small_components.py::test_open_group_store: one rank of a gloo job."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch.distributed as dist
from torch.distributed import TCPStore

from torchft_b200.bench_support import open_group_store


def main() -> None:
    rank, world, shard = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[4]}", rank=rank, world_size=world)
    group_id, group_rank = rank // shard, rank % shard
    server, port = open_group_store(world, group_id, group_rank)
    client = server if server is not None else TCPStore("127.0.0.1", port, is_master=False, wait_for_workers=False)
    if group_rank == 0:
        client.set("who", f"group{group_id}")
    dist.barrier()
    print(json.dumps({"rank": rank, "group": group_id, "port": port, "who": client.get("who").decode()}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
