#!/usr/bin/env python
"""Live-recovery benchmark: two replica groups train the same Llama model fault-tolerantly; every
group is ``--shard`` GPUs with FSDP-style sharding inside (``--shard 4`` on eight GPUs is the
2 x FSDP-4 layout of the Llama-3 8B job, ``--shard 1`` needs two GPUs).  Replica group 1 leaves
between two steps, is started again with fresh weights, and heals from group 0 while group 0
keeps training: every rank of the restarted group pulls its own shards of the weights and AdamW
moments from the same-numbered rank of the healthy group, the ranks in parallel.

    python bench_heal.py --model llama3-8b --seq-len 8192 --shard 4 --leave-at 6

Reported (one JSON line): ``heal_step_s`` the restarted group's first step (quorum, state transfer,
forward/backward, commit; max over its ranks), ``quorum_to_commit_s`` the same measured from the
moment the quorum that admits it is issued, ``state_gb`` / ``copy_gbs`` (bytes moved and the
device-timed rate of the copy kernel, per rank and summed), ``transfer_s`` (metadata fetch + copy);
for the survivor its ordinary step time, the step in which it served the checkpoint, and the host
phases of that step; ``lost_steps`` is the number of steps the survivor failed to commit (0 when
recovery is clean).  The leaving group exits between steps with nothing in flight; nothing here
faults a GPU.  ``--impl reference`` runs the same scenario on the unmodified reference
(``baseline/reference_heal.py``: reference Manager, ProcessGroupNCCL and PGTransport, torchtitan
Llama under FSDP2).
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import subprocess
import sys
import time
from datetime import timedelta

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def worker(a) -> int:
    import torch
    import torch.distributed as dist
    from torch.distributed import TCPStore

    from torchft_b200 import Manager
    from torchft_b200.checkpointing.p2p_transport import P2PTransport
    from torchft_b200.models.llama import CONFIGS
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer
    from torchft_b200.parallel.shard_comm import LocalShardComm
    from torchft_b200.parallel.team import ProcessGroupB200

    torch.cuda.set_device(a.gpu)
    dev = torch.device("cuda", a.gpu)
    cfg = CONFIGS[a.model]
    B, S = 1, a.seq_len
    timeout = timedelta(seconds=60)
    shard, gr = a.shard, a.group_rank
    store = None
    shard_comm = LocalShardComm()
    if shard > 1:
        # the group is its own torch.distributed world, as under one torchrun per replica group
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{a.group_port}", rank=gr, world_size=shard,
                                device_id=dev)
        from torchft_b200.parallel.team import PeerShardComm

        pbytes = sum(cfg.unit_numel(u) for u in range(cfg.n_units)) * 2
        shard_comm = PeerShardComm(dist.group.WORLD, dev, arena_bytes=pbytes // shard + (5 << 30))
        store_port = a.group_port
    else:
        store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
        store_port = store.port
    # gradient shards live in the replica group's arena so that the allreduce runs in place
    grad_bytes = sum(cfg.unit_numel(u) for u in range(cfg.n_units)) * 2 // shard
    pg = ProcessGroupB200(timeout=timeout, arena_bytes=grad_bytes + (64 << 20) + 300 * cfg.n_units, device=dev)
    # incoming tensors land in place in this replica's own buffers (the state is most of the GPU's memory)
    transport = P2PTransport(timeout=timeout, device=dev, state_dict=lambda: manager._manager_state_dict())
    manager = Manager(
        pg=pg, min_replica_size=1, load_state_dict=None, state_dict=None, replica_id=f"heal_rep{a.replica}",
        store_addr="127.0.0.1", store_port=store_port, rank=gr, world_size=shard, lighthouse_addr=a.lighthouse, port=0,
        hostname="127.0.0.1", timeout=timeout, quorum_timeout=timedelta(seconds=120), connect_timeout=timedelta(seconds=30),
        checkpoint_transport=transport, use_async_quorum=False, init_sync=False)
    # a restarted replica starts from different weights: only healing can make it agree with the survivor
    trainer = ShardedLlamaTrainer(cfg, B, S, dev, shard_comm=shard_comm, manager=manager, seed=1234 + 77 * a.generation,
                                  replica_alloc=pg.alloc, logit_chunks=1)
    manager.register_state_dict_fn("trainer", trainer.load_state_dict, trainer.state_dict)
    g = torch.Generator().manual_seed(5 + gr)
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
        # train_step, taken apart so that the parts of a slow step can be told from one another (the device is
        # drained between the parts, which a plain train_step does not do)
        manager.start_quorum()  # synchronous quorum: reconfiguration, serving and healing happen in here
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        loss = trainer.forward_backward(tokens[:, :-1], tokens[:, 1:])
        trainer._finish_comm()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        trainer._check_shard_team()
        ok = manager.should_commit()
        t3 = time.perf_counter()
        if ok:
            trainer.optimizer_step()
        torch.cuda.synchronize()
        t4 = time.perf_counter()
        dt = t4 - t0
        n = manager.num_participants()
        committed = manager.current_step() > before
        if not committed:
            commits_failed += 1
        phases = {k: round(v, 4) for k, v in (getattr(manager, "last_quorum_phases", {}) or {}).items()}
        phases.update({"start_quorum_s": round(t1 - t0, 4), "forward_backward_s": round(t2 - t1, 4),
                       "should_commit_s": round(t3 - t2, 4), "optimizer_s": round(t4 - t3, 4)})
        records.append({"step": manager.current_step(), "s": round(dt, 4), "participants": n, "loss": round(float(loss), 4),
                        "healed": bool(transport.last_recv) and len(records) == 0,
                        "t_end": time.time(), "phases": phases})
        if a.leave_at < 0 and step >= a.hold and rejoined_at is None:
            if n >= 2:
                rejoined_at = manager.current_step()
            elif time.time() - t_wait > 400:
                print(json.dumps({"replica": a.replica, "error": "peer never (re)joined"}), flush=True)
                os._exit(3)
    torch.cuda.synchronize()
    checksum = float(sum(m.double().sum().item() for m in trainer.master))
    print(json.dumps({"replica": a.replica, "generation": a.generation, "group_rank": gr, "records": records,
                      "last_recv": transport.last_recv, "commits_failed": commits_failed, "checksum": checksum,
                      "errored": str(pg.errored())}), flush=True)
    manager.shutdown(wait=False)
    os._exit(0)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launcher(a) -> int:
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if a.impl == "reference":
        sys.path.insert(0, os.path.join(REPO, "baseline"))
        sys.path.remove(REPO)
        import torchft_standin as cp

        worker_file = os.path.join(REPO, "baseline", "reference_heal.py")
        lh = cp.LighthouseServer("[::]:0", 1, join_timeout_ms=200, quorum_tick_ms=20, heartbeat_timeout_ms=1000)
    else:
        from torchft_b200._ftcp import LighthouseServer

        worker_file = os.path.abspath(__file__)
        lh = LighthouseServer("[::]:0", 1, join_timeout_ms=200, quorum_tick_ms=20, heartbeat_timeout_ms=1000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    shard = a.shard

    def spawn_group(replica, generation, leave_at, hold):
        port = _free_port()
        procs = []
        for r in range(shard):
            cmd = [sys.executable, worker_file, "--worker", "--replica", str(replica), "--gpu", str(replica * shard + r),
                   "--group-rank", str(r), "--shard", str(shard), "--group-port", str(port),
                   "--generation", str(generation), "--lighthouse", addr, "--model", a.model, "--seq-len", str(a.seq_len),
                   "--leave-at", str(leave_at), "--hold", str(hold), "--after", str(a.after)]
            procs.append(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env))
        return procs

    def result(proc, timeout):
        out, err = proc.communicate(timeout=timeout)
        lines = [l for l in out.splitlines() if l.startswith("{")]
        if proc.returncode != 0 or not lines:
            raise RuntimeError(f"worker rc={proc.returncode}\n{out[-1500:]}\n{err[-3000:]}")
        return json.loads(lines[-1])

    procs = []
    try:
        g0 = spawn_group(0, 0, -1, a.leave_at + 1)
        g1 = spawn_group(1, 0, a.leave_at, 0)
        procs += g0 + g1
        for p in g1:
            rc = p.wait(timeout=a.timeout)
            if rc != 17:
                raise RuntimeError(f"a rank of group 1 ended with rc={rc}: {p.stderr.read()[-3000:]}")
        t_restart = time.time()
        g1b = spawn_group(1, 1, -1, 0)
        procs += g1b
        r0 = [result(p, a.timeout) for p in g0]
        r1 = [result(p, a.timeout) for p in g1b]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()
    heal_s = max(r["records"][0]["s"] for r in r1)
    recv = [r["last_recv"] or {} for r in r1]
    total_bytes = sum(x.get("bytes", 0.0) for x in recv)
    copy_ms = max((x.get("copy_ms", 0.0) for x in recv), default=0.0)
    transfer_s = max((x.get("total_s", 0.0) for x in recv), default=0.0)
    state_bytes = max((r.get("state_bytes", 0) for r in r1), default=0)
    if total_bytes == 0 and state_bytes:
        total_bytes = float(sum(r.get("state_bytes", 0) for r in r1))
    rec0 = r0[0]["records"]
    solo = [r["s"] for r in rec0 if r["participants"] == 1]
    duo = [r["s"] for r in rec0 if r["participants"] == 2]
    # the survivor's step in which it served the checkpoint: the first one with two participants after it ran alone
    first_solo = next((i for i, r in enumerate(rec0) if r["participants"] == 1), len(rec0))
    serve = next((r for r in rec0[first_solo:] if r["participants"] == 2), None)
    duo = [r["s"] for r in rec0[first_solo:] if r["participants"] == 2 and r is not serve] or duo
    # quorum-to-commit of the healed group: from the end of the survivor's last solo step (the quorum that admits
    # the newcomer is issued in the step that follows) to the end of the healed group's first step
    last_solo_end = max((r["t_end"] for r in rec0 if r["participants"] == 1), default=None)
    healed_end = max(r["records"][0]["t_end"] for r in r1)
    sums0 = sorted(r["checksum"] for r in r0)
    sums1 = sorted(r["checksum"] for r in r1)
    same = all(abs(x - y) <= 1e-6 * max(1.0, abs(x)) for x, y in zip(sums0, sums1))
    print(json.dumps({
        "metric": "live recovery: heal time of a restarted replica group",
        "impl": a.impl,
        "heal_step_s": heal_s,
        "quorum_to_commit_s": round(healed_end - last_solo_end, 3) if last_solo_end else None,
        "transfer_s": round(transfer_s, 4),
        "state_gb": round(total_bytes / 1e9, 3),
        "state_gb_per_rank": round(total_bytes / 1e9 / shard, 3),
        "copy_ms": round(copy_ms, 3),
        "copy_gbs_per_rank": round((total_bytes / shard) / 1e6 / copy_ms, 1) if copy_ms else None,
        "copy_gbs_total": round(total_bytes / 1e6 / copy_ms, 1) if copy_ms else None,
        "healed_step_phases": max((r["records"][0] for r in r1), key=lambda x: x["s"]).get("phases"),
        "survivor_step_s": {"alone_median": sorted(solo)[len(solo) // 2] if solo else None,
                            "with_peer_median": sorted(duo)[len(duo) // 2] if duo else None,
                            "serving_step": serve["s"] if serve else None,
                            "serving_step_phases": serve.get("phases") if serve else None,
                            "max": max(r["s"] for r in rec0)},
        "lost_steps": max(r["commits_failed"] for r in r0), "replicas_equal_after": same,
        "process_restart_to_result_s": round(time.time() - t_restart, 2),
        "config": {"model": a.model, "seq_len": a.seq_len, "groups": f"2 x {shard} GPU", "leave_at_step": a.leave_at,
                   "transport": "reference PGTransport over ProcessGroupNCCL" if a.impl == "reference"
                   else "peer-memory copy kernel (P2PTransport)"},
    }))
    return 0 if same else 1


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--worker", action="store_true")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--replica", type=int, default=0)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--group-rank", type=int, default=0)
    ap.add_argument("--shard", type=int, default=1, help="GPUs per replica group (2 x shard GPUs are used)")
    ap.add_argument("--group-port", type=int, default=0)
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
