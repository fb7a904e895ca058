#!/usr/bin/env python
"""Streaming-DiLoCo benchmark: N replica groups of one GPU each train a Llama-3-style 1B
decoder (seq 2048, micro-batch 8, bf16 compute, fp32 master weights, AdamW inside) and
synchronise one of F fragments every H/F inner steps with fp8 pseudo-gradients and a
Nesterov outer step.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29544 bench_diloco.py --sync-every 100 --fragments 4 --windows 2

Prints one JSON line on rank 0.  ``outer_sync_ms`` is the time the training stream loses to one
fragment synchronisation (quorum, pseudo-gradient exchange, commit vote, outer update, bf16
refresh), CUDA-event timed, mean over the timed synchronisations, MAX over ranks: it includes
the wait for the slowest group, which is time the job really loses.  Beside it:
``arrival_spread_ms`` (how far apart the groups reach a synchronisation, from a host timestamp
taken when each group's stream has drained), ``outer_sync_work_ms`` (the same event timing on the
rank that arrived last and so waited for nobody) and ``sync_step_excess_ms`` (what the steps that
carry a synchronisation cost beyond the median plain step: the definition the reference arm
uses, so that the two arms compare like with like).  ``tokens_per_s`` is the job's aggregate over
the timed windows, synchronisations included.  ``--no-quantize`` sends fp32 instead of fp8.
``--impl reference`` runs the unmodified reference (``baseline/reference_diloco.py``).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-1b")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-backup", default="cuda", choices=["cuda", "cpu"],
                    help="reference arm: where its DiLoCo keeps the global weights (its default is pinned host "
                         "memory; device memory is the faster of its two settings)")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--sync-every", type=int, default=100, help="H: inner steps per full round of fragments")
    ap.add_argument("--fragments", type=int, default=4)
    ap.add_argument("--delay", type=int, default=0, help="fragment_sync_delay (inner steps of overlap)")
    ap.add_argument("--alpha", type=float, default=0.0, help="fragment_update_alpha")
    ap.add_argument("--windows", type=int, default=1, help="timed rounds of H inner steps (after one warm-up round)")
    ap.add_argument("--no-quantize", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(REPO, "baseline"))
        sys.path.remove(REPO)  # the product package stays out of the reference process
        import reference_diloco

        return reference_diloco.main(args)

    import torch
    import torch.distributed as dist

    from torchft_b200.bench_support import make_ft_manager
    from torchft_b200.models.llama import CONFIGS
    from torchft_b200.ops import _native as N
    from torchft_b200.parallel.diloco import EngineDiLoCo
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    cfg = CONFIGS[args.model]
    B, S = args.micro_batch, args.seq_len
    trainer = ShardedLlamaTrainer(cfg, B, S, device, seed=1234, logit_chunks=1)
    lighthouse, manager = make_ft_manager(rank, world, n_groups=world, shard=1, group_id=rank, group_rank=0,
                                          device=device, arena_bytes=0, use_async_quorum=False)
    manager.register_state_dict_fn("trainer", trainer.load_state_dict, trainer.state_dict)
    diloco = EngineDiLoCo(trainer, manager, n_fragments=args.fragments, sync_every=args.sync_every,
                          should_quantize=not args.no_quantize, fragment_sync_delay=args.delay,
                          fragment_update_alpha=args.alpha, record_timing=True)

    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    host_tokens = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).pin_memory()
    tokens = torch.empty(B, S + 1, dtype=torch.long, device=device)

    marks = []

    def run_round(timed: bool = False) -> float:
        loss = None
        for _ in range(args.sync_every):
            tokens.copy_(host_tokens, non_blocking=True)
            loss = diloco.train_step(tokens[:, :-1], tokens[:, 1:])
            if timed:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append(ev)
        return float(loss)

    run_round()  # warm-up: every fragment synchronises once
    diloco.timings.clear()
    diloco.exchange_timings.clear()
    diloco.arrival_times()
    diloco.arrivals.clear()
    commits0 = diloco.commits
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    l0 = N.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    marks.append(e0)
    last_loss = 0.0
    for _ in range(args.windows):
        last_loss = run_round(timed=True)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    total_ms = e0.elapsed_time(e1)
    launches = N.launch_count - l0
    syncs = [sum(a.elapsed_time(b) for a, b in pairs) for pairs in diloco.timings]
    sync_ms = sum(syncs) / max(1, len(syncs))
    exch = [a.elapsed_time(b) for a, b in diloco.exchange_timings]
    exch_ms = sum(exch) / max(1, len(exch))
    # the same definition as the reference arm: cost of the steps that carry a synchronisation beyond a plain step
    step_ms = [a.elapsed_time(b) for a, b in zip(marks[:-1], marks[1:])]
    every = args.sync_every // args.fragments
    special = {i for i in range(len(step_ms)) if (i % every) + 1 in (every, every - args.delay)}
    plain = sorted(ms for i, ms in enumerate(step_ms) if i not in special)
    median_step = plain[len(plain) // 2] if plain else 0.0
    excess_ms = sum(step_ms[i] - median_step for i in special) / max(1, len(step_ms) // every)
    stats = torch.tensor([total_ms, sync_ms, exch_ms, excess_ms], dtype=torch.float64, device=device)
    lo = stats.clone()
    # when did each group reach each synchronisation (monotonic clock of the one host, stream drained)?
    arr = torch.tensor(diloco.arrival_times(), dtype=torch.float64, device=device)
    arr_hi, arr_lo = arr.clone(), arr.clone()
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(arr_hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(arr_lo, op=dist.ReduceOp.MIN)
    spread_ms = float((arr_hi - arr_lo).mean().item()) * 1e3 if arr.numel() else 0.0
    total_ms, sync_ms, exch_ms, excess_ms = (float(x) for x in stats.tolist())
    # the rank that reaches a synchronisation last does not wait for anybody: its times are the work alone
    sync_ms_min, exch_ms_min = float(lo[1]), float(lo[2])
    committed = diloco.commits - commits0
    steps = args.windows * args.sync_every
    frag_elems = [sum(trainer.shard_numel[u] for u in f.units) for f in diloco.fragments]
    if rank == 0:
        print(json.dumps({
            "metric": "streaming DiLoCo outer sync ms; tokens/s",
            "impl": "ours",
            "outer_sync_ms": round(sync_ms, 3),
            "arrival_spread_ms": round(spread_ms, 3),
            "outer_sync_work_ms": round(sync_ms_min, 3),
            "sync_step_excess_ms": round(excess_ms, 3),
            "exchange_kernel_ms": round(exch_ms, 3),
            "exchange_kernel_ms_min_over_ranks": round(exch_ms_min, 3),
            "tokens_per_s": round(world * B * S * steps / (total_ms / 1e3), 1),
            "ms_per_inner_step": round((total_ms - sync_ms * len(syncs)) / steps, 3),
            "n_gpus": world, "inner_steps": steps, "syncs_timed": len(syncs), "syncs_committed": committed,
            "fragment_melems": [round(n / 1e6, 1) for n in frag_elems],
            "wire": "fp32" if args.no_quantize else "fp8 e4m3, 128-element blocks",
            "gpu_launches": launches, "final_loss": round(last_loss, 4), "dtype": "bf16", "data": "synthetic",
            "config": {"model": args.model, "seq_len": S, "micro_batch": B, "sync_every": args.sync_every,
                       "fragments": args.fragments, "fragment_sync_delay": args.delay,
                       "fragment_update_alpha": args.alpha, "parallelism": f"{world} groups x 1 GPU"},
        }))
    manager.shutdown(wait=False)
    if lighthouse is not None:
        lighthouse.shutdown()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
