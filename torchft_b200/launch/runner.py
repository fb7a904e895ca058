"""Single-box job runner and punisher.

``Runner`` keeps ``num_groups`` replica groups alive: each group is one ``torchrun``
subprocess (its own rendezvous port, ``REPLICA_GROUP_ID`` / ``NUM_REPLICA_GROUPS`` /
``TORCHFT_LIGHTHOUSE`` in the environment, a slice of the visible GPUs) and is relaunched
when it exits, up to ``max_restarts`` times -- what the reference does with Slurm jobs in
torchft/examples/slurm/runner.py:112-143 and with actors in
examples/monarch/train_distributed.py:67-312.  ``Punisher`` is the chaos side
(torchft/examples/slurm/punisher.py:15-45): ``kill_one``, ``kill_all`` and ``kill_loop``
with a mean time between failures; it signals the groups' process groups, i.e. failures
are always injected on the host.

    python -m torchft_b200.launch.runner --groups 2 --gpus-per-group 4 -- train_hsdp.py --model llama3-1b
    python -m torchft_b200.launch.runner punish --pid-file /tmp/ftb200_runner.json kill_loop --mtbf-secs 30
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


@dataclass
class GroupProc:
    group_id: int
    proc: Optional[subprocess.Popen] = None
    restarts: int = 0
    started: float = 0.0


@dataclass
class Runner:
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

    def __post_init__(self) -> None:
        self._lighthouse: Optional[LighthouseServer] = None
        self._groups = [GroupProc(i) for i in range(self.num_groups)]

    def _env(self, g: int) -> Dict[str, str]:
        env = dict(os.environ)
        env.update(self.extra_env)
        env["REPLICA_GROUP_ID"] = str(g)
        env["NUM_REPLICA_GROUPS"] = str(self.num_groups)
        env["TORCHFT_LIGHTHOUSE"] = self.lighthouse_addr or ""
        first = g * self.gpus_per_group
        env["CUDA_VISIBLE_DEVICES"] = ",".join(str(first + i) for i in range(self.gpus_per_group))
        return env

    def _launch(self, gp: GroupProc) -> None:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={self.gpus_per_group}",
               "--master-addr", "127.0.0.1", "--master-port", str(self.base_port + gp.group_id), *self.script_args]
        gp.proc = subprocess.Popen(cmd, env=self._env(gp.group_id), start_new_session=True)
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
                        continue
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
                    os.killpg(gp.proc.pid, signal.SIGTERM)
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
        os.killpg(pids[g], signal.SIGKILL)
        print(f"[punisher] killed group {g} (pgid {pids[g]})", flush=True)
        return g

    def kill_all(self) -> None:
        for g, pid in self._pids().items():
            os.killpg(pid, signal.SIGKILL)

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
        ap.add_argument("action", choices=["kill_one", "kill_all", "kill_loop"])
        ap.add_argument("--num-failures", type=int, default=10)
        ap.add_argument("--mtbf-secs", type=float, default=30.0)
        a = ap.parse_args(argv[1:])
        p = Punisher(a.pid_file)
        {"kill_one": p.kill_one, "kill_all": p.kill_all, "kill_loop": lambda: p.kill_loop(a.num_failures, a.mtbf_secs)}[a.action]()
        return 0
    ap = argparse.ArgumentParser(prog="runner")
    ap.add_argument("--groups", type=int, default=2)
    ap.add_argument("--gpus-per-group", type=int, default=1)
    ap.add_argument("--base-port", type=int, default=29600)
    ap.add_argument("--max-restarts", type=int, default=16)
    ap.add_argument("--min-replicas", type=int, default=1)
    ap.add_argument("--lighthouse", default=None)
    ap.add_argument("--pid-file", default="/tmp/ftb200_runner.json")
    ap.add_argument("script", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    script = [s for s in a.script if s != "--"]
    return Runner(script, a.groups, a.gpus_per_group, a.base_port, a.max_restarts, a.min_replicas, a.lighthouse, a.pid_file).run()


if __name__ == "__main__":
    sys.exit(main())
