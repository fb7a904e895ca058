"""Test harness for end-to-end fault-tolerance tests on one host.

A *replica group* is a thread (or a pool of ``world_size`` threads) with its own
TCPStore; the lighthouse runs in-process.  Failures are injected on the host: a train
loop raises :class:`InjectedFailure` at a chosen (replica, step) and the group restarts
from scratch, or the next allreduce's future is made to fail.
"""
from __future__ import annotations

import threading
from concurrent.futures import ThreadPoolExecutor, as_completed
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Set, Tuple

import torch
import torch.distributed as dist

from torchft_b200.process_group import FakeProcessGroupWrapper


class InjectedFailure(Exception):
    pass


class EventInjector:
    def __init__(self) -> None:
        self._lock = threading.Lock()
        self._fail: Set[Tuple[int, int, int]] = set()
        self._fail_allreduce: Set[Tuple[int, int, int]] = set()
        self._barriers: Dict[Tuple[int, int, int], threading.Barrier] = {}
        self._gates: Set[Tuple[int, int]] = set()
        self.rejoined = threading.Event()
        self.count = 0

    def fail_at(self, replica: int, step: int, rank: int = 0) -> "EventInjector":
        self._fail.add((replica, rank, step))
        return self

    def fail_allreduce_at(self, replica: int, step: int, rank: int = 0) -> "EventInjector":
        self._fail_allreduce.add((replica, rank, step))
        return self

    def gate_until_rejoin(self, replica: int, step: int) -> "EventInjector":
        """``replica`` pauses at the first check at or after ``step`` until a restarted peer
        has come back (keeps a fast survivor from finishing before the restart happens)."""
        self._gates.add((replica, step))
        return self

    def notify_restarted(self) -> None:
        self.rejoined.set()

    def barrier_at(self, replica: int, step: int, barrier: threading.Barrier, rank: int = 0) -> "EventInjector":
        self._barriers[(replica, rank, step)] = barrier
        return self

    def check(self, replica: int, rank: int, step: int, pg: Optional[FakeProcessGroupWrapper] = None) -> None:
        key = (replica, rank, step)
        with self._lock:
            # a replica that healed past the requested step still gets its failure: first check at or after it
            due = [k for k in self._fail if k[0] == replica and k[1] == rank and step >= k[2]]
            fail = bool(due)
            for k in due:
                self._fail.discard(k)
            due = [k for k in self._fail_allreduce if k[0] == replica and k[1] == rank and step >= k[2]]
            far = bool(due)
            for k in due:
                self._fail_allreduce.discard(k)
            bar = self._barriers.pop(key, None)
            if fail or far:
                self.count += 1
        gate = [g for g in self._gates if g[0] == replica and step >= g[1]]
        if gate:
            for g in gate:
                self._gates.discard(g)
            self.rejoined.wait(timeout=3)  # bounded: the peer may be the one that is waiting for us
        if fail:
            raise InjectedFailure(f"injected failure replica={replica} rank={rank} step={step}")
        if far:
            assert pg is not None
            pg.report_future_error(RuntimeError("injected allreduce failure"))
        if bar is not None:
            bar.wait(timeout=60)


@dataclass
class Runner:
    replica_id: int
    lighthouse_address: str
    injector: EventInjector
    train_loop: Callable[..., Dict[str, Any]]
    num_replicas: int = 2
    world_size: int = 1
    attempts: int = 3
    manager_args: Dict[str, Any] = field(default_factory=dict)
    train_loop_args: Dict[str, Any] = field(default_factory=dict)

    def _replica_main(self) -> List[Dict[str, Any]]:
        store = dist.TCPStore(host_name="localhost", port=0, is_master=True, wait_for_workers=False)
        with ThreadPoolExecutor(max_workers=self.world_size, thread_name_prefix=f"replica{self.replica_id}") as ex:
            futs = [ex.submit(self.train_loop, rank=r, store_port=store.port, runner=self) for r in range(self.world_size)]
            for f in as_completed(futs):
                f.result()  # propagate the first failure promptly
            return [f.result() for f in futs]

    def run_replica(self) -> List[Dict[str, Any]]:
        for attempt in range(self.attempts):
            if attempt > 0:
                self.injector.notify_restarted()
            try:
                return self._replica_main()
            except InjectedFailure as e:
                print(f"replica {self.replica_id} attempt {attempt}: {e}")
                continue
        raise RuntimeError("ran out of attempts")


def run_replicas(runners: List[Runner], timeout: float = 180) -> List[List[Dict[str, Any]]]:
    with ThreadPoolExecutor(max_workers=len(runners)) as ex:
        futs = [ex.submit(r.run_replica) for r in runners]
        return [f.result(timeout=timeout) for f in futs]
