"""Single-box job runner and punisher.

``Runner`` keeps ``num_groups`` replica groups alive: each group is one ``torchrun``
subprocess (its own rendezvous port, ``REPLICA_GROUP_ID`` / ``NUM_REPLICA_GROUPS`` /
``TORCHFT_LIGHTHOUSE`` in the environment, a slice of the visible GPUs) and is relaunched
when it exits, up to ``max_restarts`` times -- what the reference does with Slurm jobs in
torchft/examples/slurm/runner.py:112-143 and with actors in
examples/monarch/train_distributed.py:67-312.  ``Punisher`` is the chaos side
(torchft/examples/slurm/punisher.py:15-45): ``kill_one``, ``kill_all`` and ``kill_loop``
with a mean time between failures, plus ``inject`` with the failure kinds of the reference's
actor-based failure controller (examples/monarch/utils/failure.py:25-136): ``kill`` (SIGKILL),
``segfault`` (SIGSEGV), ``hang`` (SIGSTOP, then SIGKILL after a while: a process that stops
answering) and ``comms`` (SIGUSR1: a trainer that called :func:`install_fault_handlers` aborts
its replica process group and latches an error, so the step fails and the group is rebuilt
without the process dying).  Failures are always injected on the host, by signalling the
launcher and every process below it.

    python -m torchft_b200.launch.runner --groups 2 --gpus-per-group 4 -- train_hsdp.py --model llama3-1b
    python -m torchft_b200.launch.runner punish --pid-file /tmp/ftb200_runner.json kill_loop --mtbf-secs 30
    python -m torchft_b200.launch.runner punish --pid-file /tmp/ftb200_runner.json inject --kind comms --group 1
"""

from __future__ import annotations

import argparse
import json
import os
import random
import signal
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .._ftcp import LighthouseServer


FAILURE_KINDS = ("kill", "segfault", "hang", "comms")


def _descendants(pid: int, max_depth: Optional[int] = None) -> List[int]:
    """Every live process below ``pid`` (down to ``max_depth`` generations), children before grandchildren.
    ``torchrun`` starts its workers in sessions of their own, so a launcher's process group does not reach
    them; the tree is read from /proc."""
    parent_of: Dict[int, int] = {}
    for name in os.listdir("/proc"):
        if not name.isdigit():
            continue
        try:
            with open(f"/proc/{name}/stat") as f:
                stat = f.read()
            parent_of[int(name)] = int(stat[stat.rindex(")") + 2:].split()[1])  # the command may hold spaces
        except (OSError, ValueError, IndexError):
            continue
    out, frontier, depth = [], [pid], 0
    while frontier and (max_depth is None or depth < max_depth):
        nxt = [c for c, p in parent_of.items() if p in frontier]
        out += nxt
        frontier = nxt
        depth += 1
    return out


def signal_tree(pid: int, sig: int, include_root: bool = True) -> List[int]:
    """Send ``sig`` to the processes below ``pid`` (deepest last) and then, if asked, to ``pid``; returns the
    pids that were signalled."""
    hit = []
    for q in _descendants(pid) + ([pid] if include_root else []):
        try:
            os.kill(q, sig)
            hit.append(q)
        except ProcessLookupError:
            pass
    return hit


def install_fault_handlers(manager) -> None:
    """Call once from a trainer's main thread: SIGUSR1 then injects a communication failure into this
    process -- the replica process group is aborted and an error is latched in ``manager``, so the
    current step does not commit and the next quorum rebuilds the group.  The process keeps running."""

    def on_comms_fault(signum, frame) -> None:
        err = RuntimeError("injected communication failure")
        try:
            manager.report_error(err)
            manager._pg.abort()
        except Exception as e:  # never let an injection take the trainer down
            print(f"[fault] injection failed: {e}", flush=True)
        print("[fault] injected communication failure", flush=True)

    signal.signal(signal.SIGUSR1, on_comms_fault)


@dataclass
class GroupProc:
    """One replica group as the runner tracks it: its launcher process, restart count and start time."""

    group_id: int
    proc: Optional[subprocess.Popen] = None
    restarts: int = 0
    started: float = 0.0


@dataclass
class Runner:
    """Supervisor of ``num_groups`` replica groups on one box.  ``run()`` hosts a lighthouse (unless
    ``lighthouse_addr`` names one), starts one ``torchrun`` per group with ``gpus_per_group`` workers on rendezvous port
    ``base_port + group``, restarts a group that exits with a non-zero status (up to ``max_restarts`` times each) or that
    stops voting on commits (``hang_timeout_secs``), and returns when every group has exited with status 0 or has run out
    of restarts.  ``pid_file`` is where the punisher finds the launchers."""

    script_args: List[str]
    num_groups: int = 2
    gpus_per_group: int = 1
    base_port: int = 29600
    max_restarts: int = 16
    min_replicas: int = 1
    lighthouse_addr: Optional[str] = None
    pid_file: Optional[str] = None
    poll_secs: float = 1.0
    extra_env: Dict[str, str] = field(default_factory=dict)
    log_dir: Optional[str] = None  # group output goes to <log_dir>/group_<g>.<restart>.log instead of this process's stdout
    # A group whose trainers have not voted on a commit for this long is killed (and then restarted like any group that
    # exits): catches processes that are alive but stuck.  The trainers' managers write a progress file per rank at
    # every commit vote (FTB200_PROGRESS_DIR, set by the runner); None disables the check.  Choose it longer than the
    # slowest step, LocalSGD/DiLoCo window or state transfer.
    hang_timeout_secs: Optional[float] = None
    startup_grace_secs: float = 120.0  # a (re)started group gets this long for its first vote (imports, rendezvous, healing)
    progress_dir: Optional[str] = None

    def __post_init__(self) -> None:
        self._lighthouse: Optional[LighthouseServer] = None
        self._groups = [GroupProc(i) for i in range(self.num_groups)]

    def _env(self, g: int) -> Dict[str, str]:
        env = dict(os.environ)
        env.update(self.extra_env)
        env["REPLICA_GROUP_ID"] = str(g)
        env["NUM_REPLICA_GROUPS"] = str(self.num_groups)
        env["TORCHFT_LIGHTHOUSE"] = self.lighthouse_addr or ""
        if self.hang_timeout_secs is not None:
            env["FTB200_PROGRESS_DIR"] = self._progress_dir()
        first = g * self.gpus_per_group
        env["CUDA_VISIBLE_DEVICES"] = ",".join(str(first + i) for i in range(self.gpus_per_group))
        return env

    def _progress_dir(self) -> str:
        if self.progress_dir is None:
            import tempfile

            self.progress_dir = tempfile.mkdtemp(prefix="ftb200_progress_")
        return self.progress_dir

    def _is_hung(self, gp: GroupProc, now: float) -> bool:
        """No commit vote for ``hang_timeout_secs``; before the first vote of this incarnation the (longer) start-up
        grace applies instead."""
        assert self.hang_timeout_secs is not None
        newest = 0.0
        d = self._progress_dir()
        for r in range(self.gpus_per_group):
            try:
                newest = max(newest, os.path.getmtime(os.path.join(d, f"group{gp.group_id}.rank{r}")))
            except OSError:
                pass
        if newest <= gp.started:  # nothing written since this incarnation started
            return now - gp.started > max(self.startup_grace_secs, self.hang_timeout_secs)
        return now - newest > self.hang_timeout_secs

    def _launch(self, gp: GroupProc) -> None:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={self.gpus_per_group}",
               "--master-addr", "127.0.0.1", "--master-port", str(self.base_port + gp.group_id), *self.script_args]
        out = None
        if self.log_dir:
            os.makedirs(self.log_dir, exist_ok=True)
            out = open(os.path.join(self.log_dir, f"group_{gp.group_id}.{gp.restarts}.log"), "w")
        gp.proc = subprocess.Popen(cmd, env=self._env(gp.group_id), start_new_session=True, stdout=out,
                                   stderr=subprocess.STDOUT if out else None)
        if out is not None:
            out.close()  # the child holds its own descriptor
        gp.started = time.time()
        self._write_pids()

    def _write_pids(self) -> None:
        if self.pid_file:
            with open(self.pid_file, "w") as f:
                json.dump({str(g.group_id): (g.proc.pid if g.proc and g.proc.poll() is None else None) for g in self._groups}, f)

    def run(self) -> int:
        """Blocks until every group has exited with status 0 (or ran out of restarts)."""
        if not self.lighthouse_addr:
            self._lighthouse = LighthouseServer("[::]:0", self.min_replicas, join_timeout_ms=1000)
            self.lighthouse_addr = "http://127.0.0.1:" + self._lighthouse.address().rsplit(":", 1)[1]
        for gp in self._groups:
            self._launch(gp)
        done: Dict[int, int] = {}
        try:
            while len(done) < self.num_groups:
                time.sleep(self.poll_secs)
                for gp in self._groups:
                    if gp.group_id in done or gp.proc is None:
                        continue
                    rc = gp.proc.poll()
                    if rc is None:
                        if self.hang_timeout_secs is not None and self._is_hung(gp, time.time()):
                            print(f"[runner] group {gp.group_id} made no progress for {self.hang_timeout_secs} s; killing it", flush=True)
                            signal_tree(gp.proc.pid, signal.SIGKILL)
                        continue
                    signal_tree(gp.proc.pid, signal.SIGKILL, include_root=False)  # workers a dead launcher left behind
                    if rc == 0:
                        done[gp.group_id] = 0
                    elif gp.restarts < self.max_restarts:
                        gp.restarts += 1
                        print(f"[runner] group {gp.group_id} exited with {rc}; restart {gp.restarts}/{self.max_restarts}", flush=True)
                        self._launch(gp)
                    else:
                        done[gp.group_id] = rc
        finally:
            for gp in self._groups:
                if gp.proc is not None and gp.proc.poll() is None:
                    signal_tree(gp.proc.pid, signal.SIGTERM)
            if self._lighthouse is not None:
                self._lighthouse.shutdown()
        return max(done.values()) if done else 1


class Punisher:
    """Kills replica groups recorded in a runner's pid file."""

    def __init__(self, pid_file: str) -> None:
        self.pid_file = pid_file

    def _pids(self) -> Dict[int, int]:
        with open(self.pid_file) as f:
            return {int(k): v for k, v in json.load(f).items() if v}

    def kill_one(self, group: Optional[int] = None) -> Optional[int]:
        pids = self._pids()
        if not pids:
            return None
        g = group if group is not None else random.choice(sorted(pids))
        signal_tree(pids[g], signal.SIGKILL)
        print(f"[punisher] killed group {g} (launcher pid {pids[g]})", flush=True)
        return g

    def kill_all(self) -> None:
        for g, pid in self._pids().items():
            signal_tree(pid, signal.SIGKILL)

    @staticmethod
    def deliver(launcher_pid: int, kind: str, hang_secs: float = 30.0) -> None:
        """One failure of ``kind`` for the group whose launcher is ``launcher_pid``: ``kill`` takes the launcher and
        everything below it, the other kinds go to the trainer processes (the launcher's children) only; a hung
        group is killed after ``hang_secs`` so that whoever supervises the launcher can replace it."""
        if kind not in FAILURE_KINDS:
            raise ValueError(f"unknown failure kind {kind!r}; expected one of {FAILURE_KINDS}")
        if kind == "kill":
            signal_tree(launcher_pid, signal.SIGKILL)
            return
        sig = {"segfault": signal.SIGSEGV, "hang": signal.SIGSTOP, "comms": signal.SIGUSR1}[kind]
        for q in _descendants(launcher_pid, max_depth=1):
            try:
                os.kill(q, sig)
            except ProcessLookupError:
                pass
        if kind == "hang":
            time.sleep(hang_secs)
            signal_tree(launcher_pid, signal.SIGKILL)

    def inject(self, kind: str, group: Optional[int] = None, hang_secs: float = 30.0) -> Optional[int]:
        """Inject one failure of ``kind`` (see :data:`FAILURE_KINDS`) into ``group`` (random when None).
        ``segfault``, ``hang`` and ``comms`` go to the trainer processes only, not to their launcher; a hung
        group is killed after ``hang_secs`` so that its launcher's supervisor can replace it."""
        if kind not in FAILURE_KINDS:
            raise ValueError(f"unknown failure kind {kind!r}; expected one of {FAILURE_KINDS}")
        if kind == "kill":
            return self.kill_one(group)
        pids = self._pids()
        if not pids:
            return None
        g = group if group is not None else random.choice(sorted(pids))
        workers = _descendants(pids[g], max_depth=1)  # the launcher's children are the trainers
        sig = {"segfault": signal.SIGSEGV, "hang": signal.SIGSTOP, "comms": signal.SIGUSR1}[kind]
        for q in workers:
            try:
                os.kill(q, sig)
            except ProcessLookupError:
                pass
        print(f"[punisher] {kind} -> group {g} (pids {workers})", flush=True)
        if kind == "hang":
            time.sleep(hang_secs)
            signal_tree(pids[g], signal.SIGKILL)
        return g

    def kill_loop(self, num_failures: int, mtbf_secs: float) -> None:
        """``num_failures`` kills, exponentially distributed gaps with mean ``mtbf_secs``."""
        for _ in range(num_failures):
            time.sleep(random.expovariate(1.0 / mtbf_secs))
            try:
                self.kill_one()
            except (ProcessLookupError, FileNotFoundError):
                pass


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "punish":
        ap = argparse.ArgumentParser(prog="runner punish")
        ap.add_argument("--pid-file", required=True)
        ap.add_argument("action", choices=["kill_one", "kill_all", "kill_loop", "inject"])
        ap.add_argument("--num-failures", type=int, default=10)
        ap.add_argument("--mtbf-secs", type=float, default=30.0)
        ap.add_argument("--kind", choices=FAILURE_KINDS, default="kill")
        ap.add_argument("--group", type=int, default=None)
        ap.add_argument("--hang-secs", type=float, default=30.0)
        a = ap.parse_args(argv[1:])
        p = Punisher(a.pid_file)
        {"kill_one": p.kill_one, "kill_all": p.kill_all, "kill_loop": lambda: p.kill_loop(a.num_failures, a.mtbf_secs),
         "inject": lambda: p.inject(a.kind, a.group, a.hang_secs)}[a.action]()
        return 0
    ap = argparse.ArgumentParser(prog="runner")
    ap.add_argument("--groups", type=int, default=2)
    ap.add_argument("--gpus-per-group", type=int, default=1)
    ap.add_argument("--base-port", type=int, default=29600)
    ap.add_argument("--max-restarts", type=int, default=16)
    ap.add_argument("--min-replicas", type=int, default=1)
    ap.add_argument("--lighthouse", default=None)
    ap.add_argument("--pid-file", default="/tmp/ftb200_runner.json")
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--hang-timeout-secs", type=float, default=None,
                    help="kill and restart a group whose trainers have not voted on a commit for this long")
    ap.add_argument("script", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    script = [s for s in a.script if s != "--"]
    return Runner(script, a.groups, a.gpus_per_group, a.base_port, a.max_restarts, a.min_replicas, a.lighthouse, a.pid_file,
                  log_dir=a.log_dir, hang_timeout_secs=a.hang_timeout_secs).run()


if __name__ == "__main__":
    sys.exit(main())
