"""Wiring used by ``bench.py`` and the HSDP example: one lighthouse per job (hosted by
global rank 0), one TCPStore per replica group (hosted by the group's rank 0), one
:class:`~torchft_b200.manager.Manager` per rank with the NVLink peer-memory replica group."""

from __future__ import annotations

from datetime import timedelta
from typing import Optional, Tuple

import torch
import torch.distributed as dist
from torch.distributed import TCPStore

from ._ftcp import LighthouseServer
from .manager import Manager


def open_group_store(world: int, group_id: int, group_rank: int) -> Tuple[Optional[TCPStore], int]:
    """One TCPStore per replica group, hosted by the group's rank 0 on an ephemeral port (fixed offsets
    from MASTER_PORT collide when two jobs run back to back on neighbouring ports); the port travels
    over the job's default process group.  Returns ``(server or None, port)``.  Collective: every rank
    of the job calls it."""
    store = None
    mine = None
    if group_rank == 0:
        store = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
        mine = (group_id, store.port)
    if world > 1:
        ports = [None] * world
        dist.all_gather_object(ports, mine)
        return store, dict(p for p in ports if p is not None)[group_id]
    assert store is not None
    return store, store.port


def make_ft_manager(rank: int, world: int, n_groups: int, shard: int, group_id: int, group_rank: int,
                    device: torch.device, arena_bytes: int = 1 << 30, min_replica_size: Optional[int] = None,
                    timeout: timedelta = timedelta(seconds=120), use_async_quorum: bool = True,
                    checkpoint_transport=None) -> Tuple[Optional[LighthouseServer], Manager]:
    """Returns ``(lighthouse or None, manager)``.  All ranks of the job must call this.  On a CUDA device the
    replica dimension is a :class:`ProcessGroupB200` (NVLink peer memory); on CPU it is Gloo, which lets the same
    scripts run without GPUs."""
    lighthouse = None
    addr = [None]
    if rank == 0:
        lighthouse = LighthouseServer("[::]:0", min_replicas=n_groups, join_timeout_ms=200, quorum_tick_ms=10)
        port = lighthouse.address().rsplit(":", 1)[1]
        addr[0] = f"http://127.0.0.1:{port}"
    if world > 1:
        dist.broadcast_object_list(addr, src=0)
    lighthouse_addr = addr[0]

    store, base_port = open_group_store(world, group_id, group_rank)

    if device.type == "cuda":
        from .parallel.team import ProcessGroupB200

        pg = ProcessGroupB200(timeout=timeout, arena_bytes=arena_bytes, device=device)
    else:
        from .process_group import ProcessGroupGloo

        pg = ProcessGroupGloo(timeout=timeout)
    manager = Manager(
        pg=pg,
        load_state_dict=None,
        state_dict=None,
        min_replica_size=min_replica_size if min_replica_size is not None else n_groups,
        use_async_quorum=use_async_quorum,
        timeout=timeout,
        quorum_timeout=timeout,
        connect_timeout=timedelta(seconds=60),
        rank=group_rank,
        world_size=shard,
        store_addr="127.0.0.1",
        store_port=base_port,
        lighthouse_addr=lighthouse_addr,
        replica_id=f"group{group_id}",
        hostname="127.0.0.1",
        init_sync=False,  # every replica initialises from the same seed
        checkpoint_transport=checkpoint_transport,
    )
    manager._bench_store = store  # keep the group's store server alive
    return lighthouse, manager
