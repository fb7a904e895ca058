#!/usr/bin/env python
"""Live-recovery benchmark: two replica groups of one GPU each train the same Llama model
fault-tolerantly (replica-dimension allreduce through peer memory).  Replica 1 leaves
between two steps, is started again with fresh weights, and heals from replica 0 over NVLink
(peer-memory checkpoint transport) while replica 0 keeps training.

    python bench_heal.py --model llama3-8b --seq-len 8192 --leave-at 6 --steps 14

Reported (one JSON line): for the restarted replica ``heal_step_s`` (its first step: quorum,
state transfer, forward/backward, commit), ``state_gb`` and ``copy_gbs`` (bytes moved and the
device-timed rate of the copy kernel), ``transfer_s`` (metadata fetch + copy); for the
survivor the step it served the checkpoint in and its ordinary step time; ``lost_steps`` is
the number of optimizer steps the survivor failed to commit (0 when recovery is clean).
The leaving replica exits between steps with nothing in flight; nothing here faults a GPU.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from datetime import timedelta

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def worker(a) -> int:
    import torch
    from torch.distributed import TCPStore

    from torchft_b200 import Manager
    from torchft_b200.checkpointing.p2p_transport import P2PTransport
    from torchft_b200.models.llama import CONFIGS
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer
    from torchft_b200.parallel.team import ProcessGroupB200

    torch.cuda.set_device(a.gpu)
    dev = torch.device("cuda", a.gpu)
    cfg = CONFIGS[a.model]
    B, S = 1, a.seq_len
    timeout = timedelta(seconds=60)
    store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
    # gradient shards live in the replica group's arena so that the allreduce runs in place
    grad_bytes = sum(cfg.unit_numel(u) for u in range(cfg.n_units)) * 2
    pg = ProcessGroupB200(timeout=timeout, arena_bytes=grad_bytes + (64 << 20) + 300 * cfg.n_units, device=dev)
    # incoming tensors land in place in this replica's own buffers (the state is most of the GPU's memory)
    transport = P2PTransport(timeout=timeout, device=dev, state_dict=lambda: manager._manager_state_dict())
    manager = Manager(
        pg=pg, min_replica_size=1, load_state_dict=None, state_dict=None, replica_id=f"heal_rep{a.replica}",
        store_addr="127.0.0.1", store_port=store.port, rank=0, world_size=1, lighthouse_addr=a.lighthouse, port=0,
        hostname="127.0.0.1", timeout=timeout, quorum_timeout=timedelta(seconds=120), connect_timeout=timedelta(seconds=30),
        checkpoint_transport=transport, use_async_quorum=False, init_sync=False)
    # a restarted replica starts from different weights: only healing can make it agree with the survivor
    trainer = ShardedLlamaTrainer(cfg, B, S, dev, manager=manager, seed=1234 + 77 * a.generation, replica_alloc=pg.alloc,
                                  logit_chunks=1)
    manager.register_state_dict_fn("trainer", trainer.load_state_dict, trainer.state_dict)
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).to(dev)

    records = []
    commits_failed = 0
    rejoined_at = None
    t_wait = time.time()
    while True:
        step = manager.current_step()
        if a.leave_at < 0 and rejoined_at is not None and step >= rejoined_at + a.after:
            break
        if a.leave_at >= 0 and step == a.leave_at:
            torch.cuda.synchronize()
            os._exit(17)  # between steps: nothing of ours is in flight
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        before = manager.current_step()
        loss = trainer.train_step(tokens[:, :-1], tokens[:, 1:])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        n = manager.num_participants()
        committed = manager.current_step() > before
        if not committed:
            commits_failed += 1
        records.append({"step": manager.current_step(), "s": round(dt, 4), "participants": n, "loss": round(float(loss), 4),
                        "healed": bool(transport.last_recv) and len(records) == 0})
        if a.leave_at < 0 and step >= a.hold and rejoined_at is None:
            if n >= 2:
                rejoined_at = manager.current_step()
            elif time.time() - t_wait > 400:
                print(json.dumps({"replica": a.replica, "error": "peer never (re)joined"}), flush=True)
                os._exit(3)
    torch.cuda.synchronize()
    checksum = float(sum(m.double().sum().item() for m in trainer.master))
    print(json.dumps({"replica": a.replica, "generation": a.generation, "records": records, "last_recv": transport.last_recv,
                      "commits_failed": commits_failed, "checksum": checksum, "errored": str(pg.errored())}), flush=True)
    manager.shutdown(wait=False)
    os._exit(0)


def launcher(a) -> int:
    from torchft_b200._ftcp import LighthouseServer

    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=200, quorum_tick_ms=20, heartbeat_timeout_ms=1000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")

    def spawn(replica, gpu, generation, leave_at, hold):
        cmd = [sys.executable, os.path.abspath(__file__), "--worker", "--replica", str(replica), "--gpu", str(gpu),
               "--generation", str(generation), "--lighthouse", addr, "--model", a.model, "--seq-len", str(a.seq_len),
               "--leave-at", str(leave_at), "--hold", str(hold), "--after", str(a.after)]
        return subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)

    def result(proc, timeout):
        out, err = proc.communicate(timeout=timeout)
        lines = [l for l in out.splitlines() if l.startswith("{")]
        if proc.returncode != 0 or not lines:
            raise RuntimeError(f"worker rc={proc.returncode}\n{out[-1500:]}\n{err[-3000:]}")
        return json.loads(lines[-1])

    procs = []
    try:
        p0 = spawn(0, 0, 0, -1, a.leave_at + 1)
        p1 = spawn(1, 1, 0, a.leave_at, 0)
        procs += [p0, p1]
        rc = p1.wait(timeout=a.timeout)
        if rc != 17:
            raise RuntimeError(f"replica 1 ended with rc={rc}: {p1.stderr.read()[-3000:]}")
        t_restart = time.time()
        p1b = spawn(1, 1, 1, -1, 0)
        procs.append(p1b)
        r0, r1 = result(p0, a.timeout), result(p1b, a.timeout)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()
    heal = r1["records"][0]
    lr = r1["last_recv"]
    solo = [r["s"] for r in r0["records"] if r["participants"] == 1]
    duo = [r["s"] for r in r0["records"] if r["participants"] == 2]
    same = abs(r0["checksum"] - r1["checksum"]) <= 1e-6 * max(1.0, abs(r0["checksum"]))
    print(json.dumps({
        "metric": "live recovery: heal time of a restarted replica group",
        "heal_step_s": heal["s"],
        "transfer_s": round(lr.get("total_s", float("nan")), 4),
        "state_gb": round(lr.get("bytes", 0.0) / 1e9, 3),
        "copy_ms": round(lr.get("copy_ms", float("nan")), 3),
        "copy_gbs": round(lr.get("bytes", 0.0) / 1e6 / max(lr.get("copy_ms", float("nan")), 1e-9), 1),
        "survivor_step_s": {"alone_median": sorted(solo)[len(solo) // 2] if solo else None,
                            "with_peer_median": sorted(duo)[len(duo) // 2] if duo else None,
                            "max": max(r["s"] for r in r0["records"])},
        "lost_steps": r0["commits_failed"], "replicas_equal_after": same,
        "process_restart_to_result_s": round(time.time() - t_restart, 2),
        "config": {"model": a.model, "seq_len": a.seq_len, "groups": "2 x 1 GPU", "leave_at_step": a.leave_at,
                   "transport": "peer-memory copy kernel (P2PTransport)"},
    }))
    return 0 if same else 1


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--worker", action="store_true")
    ap.add_argument("--replica", type=int, default=0)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--generation", type=int, default=0)
    ap.add_argument("--lighthouse", default="")
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--leave-at", type=int, default=5)
    ap.add_argument("--hold", type=int, default=0, help="(worker) first step at which to start waiting for a peer")
    ap.add_argument("--after", type=int, default=4, help="steps to run together after the rejoin")
    ap.add_argument("--timeout", type=float, default=600.0)
    a = ap.parse_args()
    return worker(a) if a.worker else launcher(a)


if __name__ == "__main__":
    sys.exit(main())
