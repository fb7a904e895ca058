"""Round-trip latency of the control plane on one host: lighthouse + N manager servers, every
manager's ranks ask for a quorum and vote on a commit ``--iters`` times.

    python -m torchft_b200.bench_control --groups 2 --ranks-per-group 4 --iters 200

Prints one JSON line with the mean and the worst time per quorum round and per commit vote
(milliseconds, as seen by rank 0 of group 0).

    python -m torchft_b200.bench_control --manager-allreduce 200 --iters 20

measures instead the host cost of the Python ``Manager``: one replica group over ``ProcessGroupGloo`` runs
``start_quorum()``, N small ``allreduce`` calls, their waits and ``should_commit()`` per step, and the line reports
microseconds per allreduce (issue and wait) and milliseconds for the two control calls."""

from __future__ import annotations

import argparse
import json
import threading
import time
from datetime import timedelta

from . import _ftcp as C


def manager_allreduce(calls: int, iters: int) -> None:
    import logging

    import torch
    from torch.distributed import TCPStore

    from .manager import Manager
    from .process_group import ProcessGroupGloo

    logging.getLogger("torchft_b200.manager").setLevel(logging.WARNING)
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=10)
    store = TCPStore("localhost", 0, is_master=True, wait_for_workers=False)
    timeout = timedelta(seconds=10)
    m = Manager(pg=ProcessGroupGloo(timeout=timeout), min_replica_size=1, load_state_dict=lambda s: None, state_dict=lambda: {},
                replica_id="bench", store_addr="localhost", store_port=store.port, rank=0, world_size=1,
                lighthouse_addr=lh.address(), port=0, hostname="localhost", timeout=timeout)
    ts = [torch.ones(16) for _ in range(calls)]
    acc = {"quorum": 0.0, "issue": 0.0, "wait": 0.0, "commit": 0.0}
    for it in range(iters + 3):
        t0 = time.perf_counter()
        m.start_quorum()
        t1 = time.perf_counter()
        works = [m.allreduce(t) for t in ts]
        t2 = time.perf_counter()
        for w in works:
            w.wait()
        t3 = time.perf_counter()
        assert m.should_commit()
        t4 = time.perf_counter()
        if it >= 3:
            for k, v in zip(acc, (t1 - t0, t2 - t1, t3 - t2, t4 - t3)):
                acc[k] += v
    m.shutdown(wait=False)
    lh.shutdown()
    print(json.dumps({"manager_allreduce_calls": calls, "iters": iters,
                      "issue_us_per_call": round(1e6 * acc["issue"] / iters / calls, 1),
                      "wait_us_per_call": round(1e6 * acc["wait"] / iters / calls, 1),
                      "start_quorum_ms": round(1e3 * acc["quorum"] / iters, 3),
                      "should_commit_ms": round(1e3 * acc["commit"] / iters, 3)}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--groups", type=int, default=2)
    ap.add_argument("--ranks-per-group", type=int, default=1)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--manager-allreduce", type=int, default=0, metavar="N",
                    help="measure the host cost of N Manager.allreduce calls per step instead")
    a = ap.parse_args()
    if a.manager_allreduce:
        manager_allreduce(a.manager_allreduce, a.iters)
        return
    lh = C.LighthouseServer("[::]:0", a.groups, join_timeout_ms=1000, quorum_tick_ms=10)
    managers = [C.ManagerServer(replica_id=f"g{g}", lighthouse_addr=lh.address(), hostname="localhost", bind="[::]:0",
                                store_addr=f"store{g}:1", world_size=a.ranks_per_group,
                                heartbeat_interval=timedelta(milliseconds=100), connect_timeout=timedelta(seconds=5),
                                quorum_retries=0) for g in range(a.groups)]
    times = {"quorum": [], "commit": []}
    barrier = threading.Barrier(a.groups * a.ranks_per_group)

    def rank_loop(g: int, r: int) -> None:
        c = C.ManagerClient(managers[g].address(), timedelta(seconds=5))
        for step in range(a.iters + 5):
            barrier.wait()
            t0 = time.perf_counter()
            c._quorum(group_rank=r, step=step, checkpoint_metadata="m", shrink_only=False, timeout=timedelta(seconds=10),
                      init_sync=False, commit_failures=0)
            t1 = time.perf_counter()
            c.should_commit(r, step, True, timedelta(seconds=10))
            t2 = time.perf_counter()
            if g == 0 and r == 0 and step >= 5:
                times["quorum"].append((t1 - t0) * 1e3)
                times["commit"].append((t2 - t1) * 1e3)

    threads = [threading.Thread(target=rank_loop, args=(g, r)) for g in range(a.groups) for r in range(a.ranks_per_group)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for m in managers:
        m.shutdown()
    lh.shutdown()
    print(json.dumps({"groups": a.groups, "ranks_per_group": a.ranks_per_group, "iters": a.iters,
                      "quorum_ms_mean": round(sum(times["quorum"]) / len(times["quorum"]), 3),
                      "quorum_ms_max": round(max(times["quorum"]), 3),
                      "should_commit_ms_mean": round(sum(times["commit"]) / len(times["commit"]), 3),
                      "should_commit_ms_max": round(max(times["commit"]), 3)}))


if __name__ == "__main__":
    main()
