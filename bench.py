#!/usr/bin/env python
"""Headline benchmark: fault-tolerant HSDP training throughput (tokens/s) of a Llama-3 8B
decoder, seq 8192, micro-batch 1 per GPU, bf16 compute with fp32 master weights + AdamW.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29533 bench.py --gpus 8 --steps 5 --warmup 3

GPU layout (replica groups x shard size): 1 -> 1x1, 2 -> 2x1, 4 -> 2x2, 8 -> 2x4.  Every
rank runs a Manager; the lighthouse lives in global rank 0.  Each step is the full
fault-tolerant step: quorum, forward/backward, reduce-scatter inside the group,
replica-dimension allreduce through the manager, commit vote, gradient clipping, AdamW.

Prints ONE JSON line on rank 0.  ``value`` is device-timed (CUDA events, max over ranks)
with inputs resident on the device; ``e2e.value`` repeats the measurement through the
public ``train_step`` API with the step's tokens copied from pinned host memory and the
loss read back to the host every step.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def _parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--shard-comm", default="peer", choices=["peer", "nccl"])
    ap.add_argument("--no-ft", action="store_true", help="run without Manager/lighthouse (debug only)")
    ap.add_argument("--attention", default=None, choices=["tcgen05", "sdpa"],
                    help="attention kernels: hand-written tcgen05 (default where the shape allows) or the library SDPA")
    ap.add_argument("--no-fused-rs", action="store_true",
                    help="run a separate reduce-scatter kernel instead of storing weight-gradient tiles straight into "
                         "the shard owners' staging from the GEMM epilogue")
    ap.add_argument("--groups", type=int, default=0, help="replica groups (default: 1, 2, 2, 2 for 1, 2, 4, 8 GPUs)")
    ap.add_argument("--ref-ac", default="auto", choices=["auto", "full", "selective", "none"],
                    help="reference arm only: activation checkpointing of the torchtitan model (auto: torchtitan's "
                         "stock per-op selective policy, the fastest setting that fits at every layout)")
    ap.add_argument("--watchdog-s", type=int, default=600,
                    help="dump every thread's stack and exit if the run has not finished after this many seconds")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def _reference_arm(args):
    """Runs the unmodified reference (``baseline/_ref/torchft``) on its stock path; see
    ``baseline/reference_arm.py``.  Nothing of this package is imported in that process."""
    sys.path.insert(0, os.path.join(REPO, "baseline"))
    sys.path.remove(REPO)  # the product package stays out of the reference process
    import reference_arm

    args.clock_sampler = ClockSampler
    return reference_arm.main(args)


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main() -> int:
    args = _parse()
    if args.impl == "reference":
        return _reference_arm(args)

    import faulthandler

    faulthandler.dump_traceback_later(args.watchdog_s, exit=True)  # a stuck run says where, then ends

    import torch
    import torch.distributed as dist

    from torchft_b200.models.llama import CONFIGS
    from torchft_b200.ops import _native as N
    from torchft_b200.ops import kernels as K
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer
    from torchft_b200.parallel.shard_comm import LocalShardComm, TorchShardComm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # convenience: relaunch under torchrun
            port = _free_port()
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")

    t_start = time.time()

    watchdog_s = float(os.environ.get("FTB200_BENCH_WATCHDOG_S", "0"))

    def phase(name: str) -> None:
        # progress on stderr: if the run is ever cut off, the log says how far it got
        print(f"[bench rank {rank}] {name} (+{time.time() - t_start:.1f}s)", file=sys.stderr, flush=True)
        if watchdog_s > 0:
            # a phase that takes longer than this prints where every Python thread of the rank stands
            import faulthandler

            faulthandler.dump_traceback_later(watchdog_s, repeat=False, file=sys.stderr)

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cfg = CONFIGS[args.model]
    B, S = args.micro_batch, args.seq_len

    n_groups = args.groups if args.groups > 0 else (1 if world == 1 else 2)
    assert world % n_groups == 0, "--groups must divide the number of GPUs"
    shard = world // n_groups
    group_id, group_rank = rank // shard, rank % shard

    lighthouse = None
    manager = None
    shard_comm = LocalShardComm()
    if world > 1:
        phase("init_process_group")
        dist.init_process_group("nccl", device_id=dev)
        if shard > 1:
            phase("shard groups")
            groups = [dist.new_group(list(range(g * shard, (g + 1) * shard))) for g in range(n_groups)]
            if args.shard_comm == "peer":
                from torchft_b200.parallel.team import PeerShardComm

                pbytes = sum(cfg.unit_numel(u) for u in range(cfg.n_units)) * 2
                shard_comm = PeerShardComm(groups[group_id], dev, arena_bytes=pbytes // shard + (5 << 30))
            else:
                shard_comm = TorchShardComm(groups[group_id])

    if not args.no_ft:
        from torchft_b200.bench_support import make_ft_manager

        phase("manager")
        grad_bytes = sum(cfg.unit_numel(u) for u in range(cfg.n_units)) * 2 // shard
        arena = 0 if n_groups == 1 else grad_bytes + (64 << 20) + 300 * cfg.n_units
        lighthouse, manager = make_ft_manager(rank, world, n_groups, shard, group_id, group_rank, dev, arena_bytes=arena)

    replica_alloc = manager._pg.alloc if (manager is not None and n_groups > 1) else None
    phase("trainer")
    # one logits chunk: the 2 GB of bf16 logits fit, and the head's wgrad then runs once with the full reduction depth
    trainer = ShardedLlamaTrainer(cfg, B, S, dev, shard_comm=shard_comm, manager=manager, seed=1234,
                                  replica_alloc=replica_alloc, logit_chunks=1, fused_reduce_scatter=not args.no_fused_rs,
                                  attention=args.attention,
                                  wgrad_stream=True if world == 1 else None)
    if manager is not None:
        manager.register_state_dict_fn("trainer", trainer.load_state_dict, trainer.state_dict)

    g = torch.Generator(device="cpu")
    g.manual_seed(1000 + rank)
    n_batches = args.steps + args.warmup
    host_tok = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).pin_memory() for _ in range(n_batches)]
    dev_tok = [t.to(dev) for t in host_tok]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up
    phase("warm-up")
    first_loss = None
    for i in range(args.warmup):
        t = dev_tok[i]
        loss = trainer.train_step(t[:, :-1], t[:, 1:])
        if first_loss is None:
            first_loss = float(loss.item())
    K.check_status(dev)

    def committed_steps() -> int:
        return manager.current_step() if manager is not None else trainer.opt_step

    def check_commits(before: int, what: str) -> int:
        """Every step of a timed region must have committed (a declined step skips the optimizer and would
        overstate tokens/s) and the replica group must not have latched an error."""
        done = committed_steps() - before
        if done != args.steps:
            raise SystemExit(f"{what}: {done} of {args.steps} steps committed")
        if manager is not None and manager._pg.errored() is not None:
            raise SystemExit(f"{what}: replica process group errored: {manager._pg.errored()}")
        return done

    torch.cuda.synchronize()
    if committed_steps() != args.warmup:
        raise SystemExit(f"warm-up: {committed_steps()} of {args.warmup} steps committed")

    # ---- device-resident timed region
    phase("timed region")
    if os.environ.get("FTB200_TIMELINE", "0") == "1":
        trainer.exposed_comm_ms()  # drop what the warm-up recorded
    sampler = ClockSampler(local_rank)
    sync_all()
    if rank == 0:
        sampler.start()
    launches0 = N.launch_count
    steps0 = committed_steps()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        t = dev_tok[args.warmup + i]
        loss = trainer.train_step(t[:, :-1], t[:, 1:])
    e1.record()
    sync_all()
    launches = N.launch_count - launches0
    exposed = trainer.exposed_comm_ms() if os.environ.get("FTB200_TIMELINE", "0") == "1" else None
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = ms.item()
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(loss.item())
    K.check_status(dev)
    commits = check_commits(steps0, "timed region")

    phase("end-to-end region")
    # ---- end-to-end region: pinned host -> device copy of the inputs and loss read-back every step
    stage = torch.empty(B, S + 1, dtype=torch.long, device=dev)
    sync_all()
    steps0 = committed_steps()
    w0 = time.perf_counter()
    e0.record()
    losses = []
    for i in range(args.steps):
        stage.copy_(host_tok[args.warmup + i], non_blocking=True)
        loss = trainer.train_step(stage[:, :-1], stage[:, 1:])
        losses.append(float(loss.item()))  # device -> host read of the step result
        if watchdog_s > 0:
            phase(f"end-to-end step {i} done")
            K.check_status(dev)
    e1.record()
    sync_all()
    wall = time.perf_counter() - w0
    ms2 = torch.tensor([max(e0.elapsed_time(e1), wall * 1e3)], device=dev)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    K.check_status(dev)
    commits += check_commits(steps0, "end-to-end region")

    tokens_per_step = world * B * S
    value = tokens_per_step * args.steps / (ms_total / 1e3)
    e2e_value = tokens_per_step * args.steps / (ms2.item() / 1e3)
    if rank == 0:
        flops = cfg.flops_per_token(S) * B * S  # per GPU per step
        out = {
            "metric": "tokens/sec FT-HSDP Llama-3 8B" if args.model == "llama3-8b" else f"tokens/sec FT-HSDP {args.model}",
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic (seeded uniform-random token ids, random-init weights)",
            "impl": "ours",
            "config": {
                "model": args.model,
                "global_batch": world * B,
                "seq_len": S,
                "parallelism": f"hsdp: {n_groups} replica group(s) x fsdp{shard}",
                "optimizer": "AdamW, fp32 master weights and moments, grad clip 1.0",
                "l2": "working set per step (>100 GB of weights, optimizer state and activations) is far larger than L2",
                "fault_tolerance": "off (debug)" if args.no_ft else "Manager quorum + should_commit every step",
                "shard_comm": args.shard_comm if shard > 1 else "none",
                "attention": type(trainer.engine.attn).__name__,
                "reduce_scatter": ("fused into the wgrad GEMM epilogue" if trainer.fused_rs else "separate kernel") if shard > 1 else "none",
            },
            "clocks": clocks,
            "e2e": {
                "value": e2e_value,
                "unit": "tokens/s",
                "h2d_bytes_per_step": B * (S + 1) * 8,
                "d2h_bytes_per_step": 4,
            },
            "gpu_launches": launches,
            "commits": commits,
            "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 1e9, 2),
            "free_mem_gb": round(torch.cuda.mem_get_info(dev)[0] / 1e9, 2),
            **({"exposed_comm_ms_per_step": {k: round(v / args.steps, 3) for k, v in exposed.items()}} if exposed else {}),
            "model_tflops_per_gpu": flops * args.steps / (ms_total / 1e3) / 1e12,
            # uniform-random targets cannot be learned: the loss stays near that of the random initialisation,
            # ln(vocab) plus half the variance of the initial logits, and drifts down only as the logits shrink
            "loss_first_step": first_loss,
            "loss": final_loss,
        }
        print(json.dumps(out), flush=True)

    if manager is not None:
        manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
