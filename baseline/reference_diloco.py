"""Reference arm of ``bench_diloco.py``: streaming DiLoCo the way a user of the reference runs it.

The unmodified reference ``torchft.local_sgd.DiLoCo`` (``torchft/local_sgd.py:570-796``) with
``should_quantize=True`` (its Triton fp8 kernels, ``torchft/quantization.py``, through
``torchft/collectives.py:297-415``), the reference ``Manager`` with a synchronous quorum and
``ProcessGroupNCCL``; the model is torchtitan's Llama-3 ``Transformer`` at the 1B size, FSDP2 on a
mesh of one GPU for bf16 compute over fp32 master weights, ``torch.optim.AdamW`` inside and
``torch.optim.SGD(lr=0.7, momentum=0.9, nesterov=True)`` per fragment outside, exactly what
``torchtitan/components/ft/manager.py`` builds.  One replica group per GPU.  The control plane is
the pure-Python stand-in of ``torchft_standin.py``.  Nothing of the product package is imported.

The cost of a fragment synchronisation is measured the same way in both arms of the benchmark:
every inner step is bracketed by CUDA events; the steps on which a synchronisation begins or
ends cost more than the median plain step, and the excess, summed per synchronisation and
averaged, is the time the training stream loses to it (max over ranks).
"""

from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

from reference_arm import _free_port, build_model, load_reference, make_manager, unavailable  # noqa: E402


def sync_excess_ms(step_ms, sync_every, fragments, delay):
    """(mean excess per synchronisation, median plain step) from per-step times.  A synchronisation touches the
    step on which it is prepared and the step on which it is performed (the same one when ``delay`` is 0)."""
    every = sync_every // fragments
    special = set()
    for i in range(len(step_ms)):
        k = (i % every) + 1
        if k == every or k == every - delay:
            special.add(i)
    plain = sorted(ms for i, ms in enumerate(step_ms) if i not in special)
    med = plain[len(plain) // 2] if plain else 0.0
    n_sync = max(1, len(step_ms) // every)
    return sum(step_ms[i] - med for i in special) / n_sync, med


def main(args) -> int:
    try:
        torchft, standin = load_reference()
    except Exception as e:  # noqa: BLE001
        return unavailable(f"reference package not importable: {type(e).__name__}: {e}")

    import torch
    import torch.distributed as dist
    import torch.nn as nn
    import torch.nn.functional as F
    from torch.distributed.device_mesh import init_device_mesh
    from torchft.local_sgd import DiLoCo

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cpu = os.environ.get("FTB200_REF_DEVICE", "cuda") == "cpu"
    if not cpu and not torch.cuda.is_available():
        return unavailable("no CUDA device visible")
    dev = torch.device("cpu") if cpu else torch.device("cuda", local_rank)
    if not cpu:
        torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(_free_port()))
    dist.init_process_group("gloo" if cpu else "nccl", rank=rank, world_size=world)
    B, S = args.micro_batch, args.seq_len
    try:
        mesh = init_device_mesh(dev.type, (world, 1), mesh_dim_names=("replica", "shard"))
        lighthouse, manager = make_manager(torchft, standin, dist, rank, world, world, 1, rank, 0, dev,
                                           use_async_quorum=False, timeout_s=300)
        torch.manual_seed(1234)
        model, margs = build_model(args.model, S, dev, mesh["shard"], "selective")
        layers = list(model.layers.values())
        nfrag = args.fragments
        per = (len(layers) + nfrag - 1) // nfrag
        fragments = []
        for i in range(nfrag):
            mods = layers[i * per:(i + 1) * per]
            if i == 0:
                mods = [model.tok_embeddings] + mods
            if i == nfrag - 1:
                mods = mods + [model.norm, model.output]
            fragments.append(nn.ModuleList(mods))
        inner = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=not cpu)
        outers = [torch.optim.SGD([p for p in f.parameters() if p.requires_grad], lr=0.7, momentum=0.9, nesterov=True)
                  for f in fragments]
        backup = None if args.ref_backup == "cpu" else dev
        quantize = not args.no_quantize

        g = torch.Generator(device="cpu").manual_seed(100 + rank)
        host_tokens = torch.randint(0, margs.vocab_size, (B, S + 1), generator=g)
        if not cpu:
            host_tokens = host_tokens.pin_memory()
        tokens = torch.empty(B, S + 1, dtype=torch.long, device=dev)

        def new_event():
            if cpu:
                return time.perf_counter()
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e

        def elapsed(a, b):
            return (b - a) * 1e3 if cpu else a.elapsed_time(b)

        with DiLoCo(manager, fragments, inner, outers, sync_every=args.sync_every, backup_device=backup,
                    should_quantize=quantize, fragment_sync_delay=args.delay,
                    fragment_update_alpha=args.alpha) as diloco_obj:
            def run_round(marks):
                loss = None
                for _ in range(args.sync_every):
                    tokens.copy_(host_tokens, non_blocking=True)
                    inner.zero_grad()
                    pred = model(tokens[:, :-1])
                    loss = F.cross_entropy(pred.flatten(0, 1).float(), tokens[:, 1:].flatten(0, 1))
                    del pred
                    loss.backward()
                    inner.step()  # the DiLoCo hooks run here
                    if marks is not None:
                        marks.append(new_event())
                return float(loss)

            warm0 = manager.current_step()
            run_round(None)  # warm-up: every fragment synchronises once (Triton kernels compile here)
            wire_note = None
            if quantize and manager.current_step() == warm0:
                # not one synchronisation committed: on this stack the reference's quantised allreduce raises in
                # alltoall_base on its non-blocking NCCL communicator ("NCCL Error 7: NCCL operation in progress"),
                # the manager swallows the error and declines every commit.  Measure the reference's working
                # path instead: fp32 pseudo-gradients through its plain allreduce.
                wire_note = ("fp32: with should_quantize=True no synchronisation committed in the warm-up round "
                             "(the reference's allreduce_quantized fails on its ProcessGroupNCCL here)")
                quantize = False
                for f in diloco_obj._fragments:
                    f.should_quantize = False
                run_round(None)
            if not cpu:
                torch.cuda.synchronize()
            if world > 1:
                dist.barrier(**({} if cpu else {"device_ids": [local_rank]}))
            step0 = manager.current_step()
            marks = [new_event()]
            last = 0.0
            for _ in range(args.windows):
                last = run_round(marks)
            if not cpu:
                torch.cuda.synchronize()
            step_ms = [elapsed(a, b) for a, b in zip(marks[:-1], marks[1:])]
            total_ms = sum(step_ms)
            excess, med = sync_excess_ms(step_ms, args.sync_every, nfrag, args.delay)
            commits = manager.current_step() - step0
        stats = torch.tensor([total_ms, excess, med], dtype=torch.float64, device=dev)
        lo = stats.clone()
        if world > 1:
            dist.all_reduce(stats, op=dist.ReduceOp.MAX)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        steps = args.windows * args.sync_every
        if rank == 0:
            print(json.dumps({
                "metric": "streaming DiLoCo outer sync ms; tokens/s",
                "impl": "reference",
                "control_plane": "pure-Python stand-in for torchft._torchft (the Rust extension cannot be built offline)",
                "outer_sync_ms": round(float(stats[1]), 3),
                "outer_sync_ms_min_over_ranks": round(float(lo[1]), 3),
                "ms_per_inner_step": round(float(stats[2]), 3),
                "tokens_per_s": round(world * B * S * steps / (float(stats[0]) / 1e3), 1),
                "n_gpus": world, "inner_steps": steps, "syncs_timed": steps // (args.sync_every // nfrag),
                "syncs_committed": commits,
                "wire": wire_note or ("fp32" if not quantize else "fp8 e4m3, per-row scales (reference Triton kernels)"),
                "final_loss": round(last, 4), "dtype": "bf16", "data": "synthetic",
                "config": {"model": args.model, "seq_len": S, "micro_batch": B, "sync_every": args.sync_every,
                           "fragments": nfrag, "fragment_sync_delay": args.delay, "fragment_update_alpha": args.alpha,
                           "parallelism": f"{world} groups x 1 GPU", "backup_device": args.ref_backup,
                           "stack": "reference torchft DiLoCo + Manager + ProcessGroupNCCL; torchtitan Llama-3 "
                                    "Transformer, FSDP2 on a one-GPU mesh, AdamW inside, Nesterov SGD outside"},
            }), flush=True)
        manager.shutdown(wait=False)
        if lighthouse is not None:
            lighthouse.shutdown()
    except Exception as e:  # noqa: BLE001
        import traceback

        traceback.print_exc()
        if rank == 0:
            unavailable(f"reference DiLoCo arm failed at {world} GPU(s): {type(e).__name__}: {e}")
        os._exit(0)
    if world > 1:
        dist.barrier(**({} if cpu else {"device_ids": [local_rank]}))
    dist.destroy_process_group()
    return 0
