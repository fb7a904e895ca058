"""Reference arm of ``bench.py``: FT-HSDP Llama-3 8B the way a user of the reference runs it.

What runs here is the *unmodified* reference Python package (a plain copy of the reference's
``torchft/`` folder under ``baseline/_ref/``, git-ignored) on its stock path:

* ``torchft.Manager`` (``torchft/manager.py:151-175``) with ``torchft.ProcessGroupNCCL``
  (``torchft/process_group.py:738-846``) as the replica-dimension group,
* ``torchft.process_group.ManagedProcessGroup`` (``torchft/process_group.py:1233-1266``)
  installed as FSDP2's all-reduce hook, which is how torchtitan realises FT-HSDP on top of
  the reference (``README.md:62-69``; ``torchtitan/components/ft/manager.py``),
* ``torchft.optim.OptimizerWrapper`` (``torchft/optim.py:24-63``): quorum at ``zero_grad``,
  commit vote at ``step``,
* torchtitan's Llama-3 ``Transformer``, its ``apply_ac`` and ``apply_fsdp`` (FSDP2
  ``fully_shard``, bf16 compute, fp32 master weights and reductions), ``torch.optim.AdamW``
  (fused), gradient clipping at 1.0; cuBLAS, SDPA and NCCL as the reference gets them.

The one part of the reference that cannot be built offline, the Rust extension
``torchft._torchft``, is replaced by the pure-Python ``torchft_standin`` next to this file.
Nothing of the product package is imported in this process: no model, kernel, engine or
native library of ``torchft_b200``.
"""

from __future__ import annotations

import json
import os
import sys
import time
from datetime import timedelta

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")

LLAMA = {
    # name: (dim, n_layers, n_heads, n_kv_heads, ffn_dim_multiplier, multiple_of, vocab)
    "llama3-8b": dict(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=1024,
                      vocab_size=128256, rope_theta=500000),
    "llama3-1b": dict(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, ffn_dim_multiplier=1.5, multiple_of=256,
                      vocab_size=128256, rope_theta=500000),
    "debug": dict(dim=256, n_layers=2, n_heads=8, n_kv_heads=4, vocab_size=512, rope_theta=500000),
}


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)
    return 0


def load_reference():
    """Imports the reference package from ``baseline/_ref`` with the stand-in control plane."""
    if not os.path.isdir(os.path.join(REF_ROOT, "torchft")):
        raise FileNotFoundError(
            "baseline/_ref/torchft is missing: copy the reference's torchft/ folder there "
            "(cp -r <reference>/torchft baseline/_ref/torchft)")
    sys.path.insert(0, HERE)
    import torchft_standin

    torchft_standin.install(REF_ROOT)
    os.environ.setdefault("TORCHFT_USE_OTEL", "false")
    import torchft  # noqa: F401 - the reference

    assert os.path.realpath(os.path.dirname(torchft.__file__)).startswith(os.path.realpath(REF_ROOT))
    return torchft, torchft_standin


def open_group_store(dist, world, group_id, group_rank):
    from torch.distributed import TCPStore

    store, mine = None, None
    if group_rank == 0:
        store = TCPStore(host_name="127.0.0.1", port=0, is_master=True, wait_for_workers=False)
        mine = (group_id, store.port)
    if world > 1:
        ports = [None] * world
        dist.all_gather_object(ports, mine)
        return store, dict(p for p in ports if p is not None)[group_id]
    return store, store.port


def make_manager(torchft, standin, dist, rank, world, n_groups, shard, group_id, group_rank, device,
                 use_async_quorum=True, timeout_s=120, checkpoint_transport=None, min_replica_size=None):
    """One lighthouse per job (global rank 0), one TCPStore per replica group, one reference Manager per rank."""
    lighthouse, addr = None, [None]
    if rank == 0:
        lighthouse = standin.LighthouseServer("[::]:0", min_replicas=n_groups, join_timeout_ms=200, quorum_tick_ms=10)
        addr[0] = f"http://127.0.0.1:{lighthouse.address().rsplit(':', 1)[1]}"
    if world > 1:
        dist.broadcast_object_list(addr, src=0)
    store, port = open_group_store(dist, world, group_id, group_rank)
    timeout = timedelta(seconds=timeout_s)
    pg = torchft.ProcessGroupNCCL(timeout=timeout) if device.type == "cuda" else torchft.ProcessGroupGloo(timeout=timeout)
    manager = torchft.Manager(
        pg=pg, load_state_dict=None, state_dict=None,
        min_replica_size=min_replica_size if min_replica_size is not None else n_groups,
        use_async_quorum=use_async_quorum, timeout=timeout, quorum_timeout=timeout,
        connect_timeout=timedelta(seconds=60), rank=group_rank, world_size=shard,
        store_addr="127.0.0.1", store_port=port, lighthouse_addr=addr[0], replica_id=f"group{group_id}",
        hostname="127.0.0.1", init_sync=False, checkpoint_transport=checkpoint_transport,
    )
    manager._bench_store = store
    return lighthouse, manager


def build_model(name, seq_len, device, shard_mesh, ac_mode):
    import torch
    from torchtitan.config.job_config import ActivationCheckpoint
    from torchtitan.models.llama3 import Transformer, TransformerModelArgs
    from torchtitan.models.llama3.infra.parallelize import apply_ac, apply_fsdp

    margs = TransformerModelArgs(max_seq_len=seq_len, **LLAMA[name])
    with torch.device("meta"):
        model = Transformer(margs)
    if ac_mode != "none":
        apply_ac(model, ActivationCheckpoint(mode=ac_mode, selective_ac_option="op"))
    apply_fsdp(model, shard_mesh, param_dtype=torch.bfloat16, reduce_dtype=torch.float32, pp_enabled=False)
    model.to_empty(device=device)
    with torch.no_grad():
        model.init_weights(buffer_device=device)
    model.train()
    return model, margs


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def main(args) -> int:
    try:
        torchft, standin = load_reference()
    except Exception as e:  # noqa: BLE001
        return unavailable(f"reference package not importable: {type(e).__name__}: {e}")

    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from torch.distributed._composable.fsdp.fully_shard import FSDPModule
    from torch.distributed.device_mesh import init_device_mesh
    from torchtitan.distributed.utils import clip_grad_norm_

    from torchft.optim import OptimizerWrapper
    from torchft.process_group import ManagedProcessGroup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cpu = os.environ.get("FTB200_REF_DEVICE", "cuda") == "cpu"  # plumbing check without GPUs
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            import subprocess

            port = _free_port()
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port),
                   os.path.join(os.path.dirname(HERE), "bench.py")] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not cpu and not torch.cuda.is_available():
        return unavailable("no CUDA device visible")

    if cpu:
        dev = torch.device("cpu")
    else:
        torch.cuda.set_device(local_rank)
        dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(_free_port()))
    # no device_id: the reference's ProcessGroup.register() (torchft/process_group.py:326-345) creates a
    # world-size-1 group of its own backend, which torch refuses on a default group bound to a device
    dist.init_process_group("gloo" if cpu else "nccl", rank=rank, world_size=world)

    n_groups = args.groups if args.groups > 0 else (1 if world == 1 else 2)
    shard = world // n_groups
    group_id, group_rank = rank // shard, rank % shard
    B, S = args.micro_batch, args.seq_len

    try:
        # the shard mesh of this replica group only: the replica dimension belongs to the manager
        mesh = init_device_mesh(dev.type, (n_groups, shard), mesh_dim_names=("replica", "shard"))
        shard_mesh = mesh["shard"]
        lighthouse, manager = make_manager(torchft, standin, dist, rank, world, n_groups, shard, group_id,
                                           group_rank, dev)
        replicate_pg = ManagedProcessGroup(manager)
        replicate_pg.register("dp_replicate")

        ac_mode = args.ref_ac
        if ac_mode == "auto":
            # torchtitan's stock Llama-3 8B setting (per-op selective checkpointing).  It fits at every
            # layout (measured peak 131 GB where the group is one GPU) and is faster than full recomputation.
            ac_mode = "selective"
        torch.manual_seed(1234)
        model, margs = build_model(args.model, S, dev, shard_mesh, ac_mode)

        def all_reduce_hook(output):
            dist.all_reduce(output, group=replicate_pg, op=dist.ReduceOp.AVG)

        for m in model.modules():
            if isinstance(m, FSDPModule):
                m.set_all_reduce_hook(all_reduce_hook)

        inner = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1,
                                  fused=not cpu)
        optim = OptimizerWrapper(manager, inner)
        params = list(model.parameters())

        def train_step(tokens, labels):
            optim.zero_grad()  # starts the quorum
            pred = model(tokens)
            loss = F.cross_entropy(pred.flatten(0, 1).float(), labels.flatten(0, 1))
            del pred
            loss.backward()
            clip_grad_norm_(params, 1.0, foreach=True)
            optim.step()  # commit vote, then AdamW
            return loss.detach()

        g = torch.Generator(device="cpu")
        g.manual_seed(1000 + rank)
        n_batches = args.steps + args.warmup
        vocab = margs.vocab_size
        host_tok = [torch.randint(0, vocab, (B, S + 1), generator=g) for _ in range(n_batches)]
        if not cpu:
            host_tok = [t.pin_memory() for t in host_tok]
        dev_tok = [t.to(dev) for t in host_tok]

        def sync_all():
            if not cpu:
                torch.cuda.synchronize()
            if world > 1:
                dist.barrier(**({} if cpu else {"device_ids": [local_rank]}))
            if not cpu:
                torch.cuda.synchronize()

        def timer():
            if cpu:
                t0 = time.perf_counter()
                return lambda: (time.perf_counter() - t0) * 1e3
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()

            def stop():
                e1.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1)
            return stop

        for i in range(args.warmup):
            t = dev_tok[i]
            loss = train_step(t[:, :-1], t[:, 1:])
        sync_all()
        step0 = manager.current_step()
        assert step0 == args.warmup, f"warm-up committed {step0} of {args.warmup} steps"

        sampler = None
        if rank == 0 and not cpu and args.clock_sampler is not None:
            sampler = args.clock_sampler(local_rank)
            sampler.start()
        stop = timer()
        for i in range(args.steps):
            t = dev_tok[args.warmup + i]
            loss = train_step(t[:, :-1], t[:, 1:])
        ms_local = stop()
        sync_all()
        ms = torch.tensor([ms_local], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        clocks = sampler.stop() if sampler is not None else None
        final_loss = float(loss.item())
        commits = manager.current_step() - step0

        # end to end: pinned host -> device copy of the tokens and loss read-back, every step
        stage = torch.empty(B, S + 1, dtype=torch.long, device=dev)
        sync_all()
        w0 = time.perf_counter()
        stop = timer()
        for i in range(args.steps):
            stage.copy_(host_tok[args.warmup + i], non_blocking=True)
            loss = train_step(stage[:, :-1], stage[:, 1:])
            float(loss.item())
        ms2_local = stop()
        sync_all()
        wall = (time.perf_counter() - w0) * 1e3
        ms2 = torch.tensor([max(ms2_local, wall)], device=dev)
        if world > 1:
            dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        commits2 = manager.current_step() - step0 - commits
        assert commits == args.steps and commits2 == args.steps, (commits, commits2)
        assert manager._pg.errored() is None

        peak_gb = 0.0 if cpu else torch.cuda.max_memory_allocated() / 1e9
        tokens_per_step = world * B * S
        if rank == 0:
            out = {
                "metric": "tokens/sec FT-HSDP Llama-3 8B" if args.model == "llama3-8b" else f"tokens/sec FT-HSDP {args.model}",
                "value": tokens_per_step * args.steps / (ms.item() / 1e3),
                "unit": "tokens/s",
                "n_gpus": world,
                "steps": args.steps,
                "warmup": args.warmup,
                "ms_per_step": ms.item() / args.steps,
                "higher_is_better": True,
                "scaling": "weak",
                "vs_baseline": None,
                "dtype": "bf16",
                "data": "synthetic (seeded uniform-random token ids, random-init weights)",
                "impl": "reference",
                "control_plane": "pure-Python stand-in for torchft._torchft (the Rust extension cannot be built offline)",
                "config": {
                    "model": args.model,
                    "global_batch": world * B,
                    "seq_len": S,
                    "parallelism": f"hsdp: {n_groups} replica group(s) x fsdp{shard}",
                    "optimizer": "torch.optim.AdamW (fused), fp32 master weights and moments, grad clip 1.0",
                    "stack": "reference torchft Manager + ProcessGroupNCCL + ManagedProcessGroup all-reduce hook + "
                             "OptimizerWrapper; torchtitan Llama-3 Transformer, FSDP2 fully_shard (bf16 compute, fp32 reduce)",
                    "activation_checkpoint": ac_mode,
                    "l2": "working set per step is far larger than L2",
                    "fault_tolerance": "Manager quorum + should_commit every step",
                },
                "clocks": clocks,
                "e2e": {
                    "value": tokens_per_step * args.steps / (ms2.item() / 1e3),
                    "unit": "tokens/s",
                    "h2d_bytes_per_step": B * (S + 1) * 8,
                    "d2h_bytes_per_step": 4,
                },
                "gpu_launches": None,
                "commits": commits + commits2,
                "peak_mem_gb": peak_gb,
                "loss": final_loss,
            }
            print(json.dumps(out), flush=True)
        manager.shutdown(wait=False)
        if lighthouse is not None:
            lighthouse.shutdown()
    except Exception as e:  # noqa: BLE001 - one N that cannot run reports why instead of a stack only
        import traceback

        traceback.print_exc()
        if rank == 0:
            unavailable(f"reference arm failed at {world} GPU(s): {type(e).__name__}: {e}")
        os._exit(0)
    if world > 1:
        dist.barrier(**({} if cpu else {"device_ids": [local_rank]}))
    dist.destroy_process_group()
    return 0
