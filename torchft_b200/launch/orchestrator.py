"""Job orchestration over *allocations*: which resources a replica group runs on is a decision of its own,
separate from restarting the group's processes.

The reference's actor-based orchestrator (examples/monarch/train_distributed.py:200-312) retries a failed replica on
the allocation it has (``PROC_ATTEMPTS`` times), then gives the allocation back and asks the scheduler for a new
one, and gives the replica up after ``MAX_ATTEMPT`` attempts; a failure controller
(examples/monarch/utils/failure.py:81-136) injects failures into running replicas.  This module is the same policy
without an actor framework:

* :class:`Allocator` hands out allocations.  :class:`GpuPoolAllocator` is the one-box scheduler: a pool of GPU
  indices cut into slices; a slice that was given back after repeated failures is quarantined, so the next
  request gets different GPUs for as long as spares exist.  :class:`SlurmAllocator` reserves nodes with ``salloc``
  and releases them with ``scancel`` (built on the commands of :mod:`torchft_b200.launch.slurm`).
* :class:`Orchestrator` runs one supervisor thread per replica group: start the group's launcher on its allocation,
  wait, on failure retry after a delay; every ``proc_attempts`` failures in a row exchange the allocation; after
  ``max_attempts`` attempts the group is abandoned (the other groups keep training: that is the point of the
  quorum).  It hosts the lighthouse unless given one, and an optional :class:`FailureController` thread injects
  the failure kinds of :mod:`torchft_b200.launch.runner` at random into running groups.

    python -m torchft_b200.launch.orchestrator --groups 2 --gpus-per-group 4 --spare-gpus 0 -- train_hsdp.py ...
"""

from __future__ import annotations

import argparse
import logging
import os
import random
import subprocess
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from .runner import FAILURE_KINDS, Punisher, signal_tree

logger = logging.getLogger(__name__)


@dataclass
class Allocation:
    """Resources one replica group runs on: an identifier, the environment that points a launcher at them and,
    for allocations made of hosts, a command prefix (``srun --jobid ...``)."""

    name: str
    env: Dict[str, str] = field(default_factory=dict)
    prefix: List[str] = field(default_factory=list)


class Allocator:
    """Source of allocations.  ``acquire`` may block until resources are free; ``release(..., failed=True)`` says
    that the group kept failing there."""

    def acquire(self, group_id: int) -> Allocation:
        raise NotImplementedError

    def release(self, allocation: Allocation, failed: bool) -> None:
        raise NotImplementedError


class GpuPoolAllocator(Allocator):
    """GPUs of one box in slices of ``gpus_per_group``.  A slice released as failed goes to the back of the queue
    behind every slice that has not failed, so a group whose GPUs look broken moves to spare GPUs if there are any
    and otherwise gets its old slice back."""

    def __init__(self, gpus: Sequence[int], gpus_per_group: int) -> None:
        if gpus_per_group < 1 or len(gpus) < gpus_per_group:
            raise ValueError("need at least one slice of GPUs")
        self._per = gpus_per_group
        self._free: List[List[int]] = [list(gpus[i:i + gpus_per_group]) for i in range(0, len(gpus) - gpus_per_group + 1, gpus_per_group)]
        self._suspect: List[List[int]] = []
        self._cv = threading.Condition()

    def acquire(self, group_id: int) -> Allocation:
        with self._cv:
            while not self._free and not self._suspect:
                self._cv.wait()
            gpus = self._free.pop(0) if self._free else self._suspect.pop(0)
        return Allocation(name="gpus-" + "-".join(map(str, gpus)),
                          env={"CUDA_VISIBLE_DEVICES": ",".join(map(str, gpus)), "FTB200_ALLOCATION_GPUS": ",".join(map(str, gpus))})

    def release(self, allocation: Allocation, failed: bool) -> None:
        gpus = [int(x) for x in allocation.env["FTB200_ALLOCATION_GPUS"].split(",")]
        with self._cv:
            (self._suspect if failed else self._free).append(gpus)
            self._cv.notify()


class SlurmAllocator(Allocator):
    """One Slurm allocation of ``nodes`` nodes per replica group (``salloc --no-shell``); the group's launcher runs
    under ``srun --jobid``.  Giving an allocation back cancels the job, so a new request lands on whatever nodes
    Slurm chooses next."""

    def __init__(self, nodes: int = 1, salloc_args: Sequence[str] = (), run: Callable[..., "subprocess.CompletedProcess"] = subprocess.run) -> None:
        self._nodes, self._args, self._run = nodes, list(salloc_args), run

    def acquire(self, group_id: int) -> Allocation:
        name = f"ft_{group_id}"
        out = self._run(["salloc", "--no-shell", f"--nodes={self._nodes}", f"--job-name={name}", *self._args],
                        capture_output=True, text=True, check=True)
        text = (out.stderr or "") + (out.stdout or "")
        job = next((tok for tok in text.replace(".", " ").split() if tok.isdigit()), None)
        if job is None:
            raise RuntimeError(f"salloc did not report a job id: {text!r}")
        return Allocation(name=f"slurm-{job}", env={"SLURM_JOB_ID": job}, prefix=["srun", f"--jobid={job}"])

    def release(self, allocation: Allocation, failed: bool) -> None:
        self._run(["scancel", allocation.env["SLURM_JOB_ID"]], capture_output=True, text=True)


@dataclass
class GroupState:
    """What the orchestrator knows about one replica group."""

    group_id: int
    attempts: int = 0
    allocations: List[str] = field(default_factory=list)
    proc: Optional[subprocess.Popen] = None
    done: bool = False
    abandoned: bool = False


class FailureController(threading.Thread):
    """Injects failures into running groups: every ``mtbf_secs`` on average one random group gets one of ``kinds``
    (see :data:`torchft_b200.launch.runner.FAILURE_KINDS`), by signalling its launcher's process tree."""

    def __init__(self, groups: Dict[int, GroupState], mtbf_secs: float, kinds: Sequence[str] = FAILURE_KINDS,
                 seed: Optional[int] = None) -> None:
        super().__init__(name="ftb200-failures", daemon=True)
        self._groups, self._mtbf, self._kinds = groups, mtbf_secs, list(kinds)
        self._rng = random.Random(seed)
        self._halt = threading.Event()
        self.injected: List[tuple] = []

    def run(self) -> None:
        while not self._halt.wait(self._rng.expovariate(1.0 / self._mtbf)):
            live = [g for g in self._groups.values() if g.proc is not None and g.proc.poll() is None]
            if not live:
                continue
            g, kind = self._rng.choice(live), self._rng.choice(self._kinds)
            assert g.proc is not None
            Punisher.deliver(g.proc.pid, kind)
            self.injected.append((time.time(), g.group_id, kind))
            logger.info("injected %s into group %d", kind, g.group_id)

    def stop(self) -> None:
        self._halt.set()


class Orchestrator:
    """Keeps ``num_groups`` replica groups running under the retry / new-allocation policy described in the module
    docstring.  ``command(group_id, allocation)`` returns the launcher command line of a group (without the
    allocation's prefix); :meth:`torchrun_command` builds the usual one."""

    def __init__(self, num_groups: int, allocator: Allocator, command: Callable[[int, Allocation], List[str]],
                 lighthouse_addr: Optional[str] = None, min_replicas: int = 1, proc_attempts: int = 4,
                 max_attempts: int = 16, retry_delay_s: float = 10.0, env: Optional[Dict[str, str]] = None,
                 log_dir: Optional[str] = None) -> None:
        self.num_groups, self.allocator, self.command = num_groups, allocator, command
        self.proc_attempts, self.max_attempts, self.retry_delay_s = proc_attempts, max_attempts, retry_delay_s
        self.env, self.log_dir = dict(env or {}), log_dir
        self.groups: Dict[int, GroupState] = {g: GroupState(g) for g in range(num_groups)}
        self._lighthouse = None
        self.lighthouse_addr = lighthouse_addr
        self._min_replicas = min_replicas
        self._stop = threading.Event()

    @staticmethod
    def torchrun_command(script_args: Sequence[str], nproc: int, base_port: int = 29600) -> Callable[[int, Allocation], List[str]]:
        def build(group_id: int, allocation: Allocation) -> List[str]:
            return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
                    "--master-addr", "127.0.0.1", f"--master-port={base_port + group_id}", *script_args]
        return build

    def _supervise(self, g: GroupState) -> None:
        allocation = self.allocator.acquire(g.group_id)
        g.allocations.append(allocation.name)
        failures_here = 0
        try:
            while not self._stop.is_set():
                if g.attempts >= self.max_attempts:
                    g.abandoned = True
                    logger.error("group %d failed %d times: giving it up", g.group_id, g.attempts)
                    return
                if failures_here and failures_here % self.proc_attempts == 0:
                    logger.warning("group %d failed %d times on %s: getting a new allocation", g.group_id, failures_here,
                                   allocation.name)
                    self.allocator.release(allocation, failed=True)
                    allocation = self.allocator.acquire(g.group_id)
                    g.allocations.append(allocation.name)
                    failures_here = 0
                if g.attempts and self._stop.wait(self.retry_delay_s):
                    return
                g.attempts += 1
                env = dict(os.environ, **self.env, **allocation.env, REPLICA_GROUP_ID=str(g.group_id),
                           NUM_REPLICA_GROUPS=str(self.num_groups), TORCHFT_LIGHTHOUSE=str(self.lighthouse_addr))
                out = None
                if self.log_dir:
                    os.makedirs(self.log_dir, exist_ok=True)
                    out = open(os.path.join(self.log_dir, f"group{g.group_id}.attempt{g.attempts}.log"), "w")
                g.proc = subprocess.Popen(allocation.prefix + self.command(g.group_id, allocation), env=env, stdout=out,
                                          stderr=subprocess.STDOUT if out else None, start_new_session=True)
                while g.proc.poll() is None:
                    if self._stop.wait(0.2):
                        signal_tree(g.proc.pid, 9)
                        return
                if out:
                    out.close()
                if g.proc.returncode == 0:
                    g.done = True
                    return
                failures_here += 1
                logger.warning("group %d exited with %s (attempt %d)", g.group_id, g.proc.returncode, g.attempts)
        finally:
            self.allocator.release(allocation, failed=False)

    def run(self, failures: Optional[FailureController] = None) -> Dict[int, GroupState]:
        """Blocks until every group has finished or been given up; returns the groups' final states."""
        if self.lighthouse_addr is None:
            from .._ftcp import LighthouseServer

            self._lighthouse = LighthouseServer("[::]:0", self._min_replicas)
            self.lighthouse_addr = "http://127.0.0.1:" + self._lighthouse.address().rsplit(":", 1)[1]
        threads = [threading.Thread(target=self._supervise, args=(g,), name=f"ftb200-group{g.group_id}", daemon=True)
                   for g in self.groups.values()]
        if failures is not None:
            failures.start()
        try:
            for t in threads:
                t.start()
            for t in threads:
                while t.is_alive():
                    t.join(0.5)
        except KeyboardInterrupt:
            self._stop.set()
            for t in threads:
                t.join(5)
        finally:
            if failures is not None:
                failures.stop()
            if self._lighthouse is not None:
                self._lighthouse.shutdown()
        return self.groups

    def stop(self) -> None:
        self._stop.set()


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--groups", type=int, default=2)
    ap.add_argument("--gpus-per-group", type=int, default=1)
    ap.add_argument("--spare-gpus", type=int, default=0, help="GPUs beyond groups x gpus-per-group that failed groups may move to")
    ap.add_argument("--proc-attempts", type=int, default=4)
    ap.add_argument("--max-attempts", type=int, default=16)
    ap.add_argument("--retry-delay-secs", type=float, default=10.0)
    ap.add_argument("--lighthouse", default=None)
    ap.add_argument("--min-replicas", type=int, default=1)
    ap.add_argument("--mtbf-secs", type=float, default=0.0, help="inject failures with this mean time between them (0: none)")
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("script", nargs=argparse.REMAINDER)
    a = ap.parse_args()
    script = a.script[1:] if a.script[:1] == ["--"] else a.script
    if not script:
        ap.error("give the training script after --")
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(message)s")
    total = a.groups * a.gpus_per_group + a.spare_gpus
    orch = Orchestrator(a.groups, GpuPoolAllocator(list(range(total)), a.gpus_per_group),
                        Orchestrator.torchrun_command(script, a.gpus_per_group), lighthouse_addr=a.lighthouse,
                        min_replicas=a.min_replicas, proc_attempts=a.proc_attempts, max_attempts=a.max_attempts,
                        retry_delay_s=a.retry_delay_secs, log_dir=a.log_dir)
    failures = FailureController(orch.groups, a.mtbf_secs) if a.mtbf_secs > 0 else None
    groups = orch.run(failures)
    return 0 if all(g.done for g in groups.values()) else 1


if __name__ == "__main__":
    sys.exit(main())
