"""Slurm helpers: keep ``ft_<id>`` jobs (one per replica group) running, and kill them.

``runner`` polls ``squeue`` every 10 s and resubmits missing replica jobs with ``sbatch
--wrap`` (torchft/examples/slurm/runner.py:112-143); ``punisher`` cancels jobs with
``scancel``: ``kill_one``, ``kill_all``, ``kill_loop --mtbf-secs`` (the sleep between
kills is drawn from an exponential distribution with that mean; the reference computes
such a value and then sleeps the mean, torchft/examples/slurm/punisher.py:43-45).
Requires the Slurm client tools on PATH.

    python -m torchft_b200.launch.slurm runner --replicas 4 --nodes-per-replica 1 -- train_hsdp.py --model llama3-8b
    python -m torchft_b200.launch.slurm punisher kill_loop --mtbf-secs 300
"""

from __future__ import annotations

import argparse
import random
import shlex
import subprocess
import time
from typing import List, Set

PREFIX = "ft_"


def _running() -> Set[str]:
    out = subprocess.run(["squeue", "--me", "-h", "-o", "%j"], capture_output=True, text=True, check=True).stdout
    return {l.strip() for l in out.splitlines() if l.strip().startswith(PREFIX)}


def _submit(replica: int, replicas: int, nodes: int, gpus: int, lighthouse: str, script: List[str]) -> None:
    inner = (f"REPLICA_GROUP_ID={replica} NUM_REPLICA_GROUPS={replicas} TORCHFT_LIGHTHOUSE={lighthouse} "
             f"torchrun --nnodes={nodes} --nproc-per-node={gpus} --rdzv_backend=c10d --rdzv_endpoint=$(hostname):29500 "
             + " ".join(shlex.quote(s) for s in script))
    subprocess.run(["sbatch", f"--job-name={PREFIX}{replica}", f"--nodes={nodes}", f"--gpus-per-node={gpus}",
                    "--wrap", inner], check=True)


def runner(replicas: int, nodes: int, gpus: int, lighthouse: str, script: List[str], poll_secs: float = 10.0) -> None:
    """Keep one Slurm job per replica group (``ft_<g>``) in the queue: every ``poll_secs`` submit the ones that are
    missing.  Runs until interrupted."""
    while True:
        alive = _running()
        for r in range(replicas):
            if f"{PREFIX}{r}" not in alive:
                print(f"[slurm runner] (re)submitting replica {r}", flush=True)
                _submit(r, replicas, nodes, gpus, lighthouse, script)
        time.sleep(poll_secs)


def kill_one() -> None:
    """``scancel`` one randomly chosen replica-group job."""
    jobs = sorted(_running())
    if jobs:
        victim = random.choice(jobs)
        print(f"[slurm punisher] scancel {victim}", flush=True)
        subprocess.run(["scancel", f"--name={victim}"], check=True)


def kill_all() -> None:
    """``scancel`` every replica-group job."""
    for j in _running():
        subprocess.run(["scancel", f"--name={j}"], check=True)


def kill_loop(num_failures: int, mtbf_secs: float) -> None:
    """``num_failures`` times: sleep an exponentially distributed time with mean ``mtbf_secs``, then ``kill_one``."""
    for _ in range(num_failures):
        time.sleep(random.expovariate(1.0 / mtbf_secs))
        kill_one()


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("runner")
    r.add_argument("--replicas", type=int, default=2)
    r.add_argument("--nodes-per-replica", type=int, default=1)
    r.add_argument("--gpus-per-node", type=int, default=8)
    r.add_argument("--lighthouse", default="http://localhost:29510")
    r.add_argument("script", nargs=argparse.REMAINDER)
    p = sub.add_parser("punisher")
    p.add_argument("action", choices=["kill_one", "kill_all", "kill_loop"])
    p.add_argument("--num-failures", type=int, default=10)
    p.add_argument("--mtbf-secs", type=float, default=300.0)
    a = ap.parse_args()
    if a.cmd == "runner":
        runner(a.replicas, a.nodes_per_replica, a.gpus_per_node, a.lighthouse, [s for s in a.script if s != "--"])
    else:
        {"kill_one": kill_one, "kill_all": kill_all, "kill_loop": lambda: kill_loop(a.num_failures, a.mtbf_secs)}[a.action]()


if __name__ == "__main__":
    main()
