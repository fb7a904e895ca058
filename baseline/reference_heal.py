"""One rank of the reference arm of ``bench_heal.py`` (started by its launcher with ``--impl reference``).

The scenario of ``bench_heal.py`` on the unmodified reference: ``torchft.Manager`` with a synchronous
quorum, ``torchft.ProcessGroupNCCL`` as the replica-dimension group and, for the state transfer,
the reference's ``PGTransport`` (``torchft/checkpointing/pg_transport.py:163-300``) in its in-place
mode, which is the faster of the reference's transports (no host hop); torchtitan's Llama-3
``Transformer`` under FSDP2 inside the replica group, ``torch.optim.AdamW``.  The restarted group
allocates its AdamW moments before it heals so that the in-place receive applies to them too.
Prints the same JSON record as the worker of ``bench_heal.py``.  Nothing of the product package is
imported.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from datetime import timedelta

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

from reference_arm import build_model, load_reference  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--worker", action="store_true")
    ap.add_argument("--replica", type=int, default=0)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--group-rank", type=int, default=0)
    ap.add_argument("--shard", type=int, default=1)
    ap.add_argument("--group-port", type=int, default=0)
    ap.add_argument("--generation", type=int, default=0)
    ap.add_argument("--lighthouse", default="")
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--leave-at", type=int, default=5)
    ap.add_argument("--hold", type=int, default=0)
    ap.add_argument("--after", type=int, default=4)
    a = ap.parse_args()

    torchft, _ = load_reference()
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from torch.distributed._composable.fsdp.fully_shard import FSDPModule
    from torch.distributed.device_mesh import init_device_mesh
    from torchtitan.distributed.utils import clip_grad_norm_

    from torchft.checkpointing.pg_transport import PGTransport
    from torchft.optim import OptimizerWrapper
    from torchft.process_group import ManagedProcessGroup

    cpu = os.environ.get("FTB200_REF_DEVICE", "cuda") == "cpu"
    dev = torch.device("cpu") if cpu else torch.device("cuda", a.gpu)
    if not cpu:
        torch.cuda.set_device(dev)
    shard, gr = a.shard, a.group_rank
    # the group is its own torch.distributed world, as under one torchrun per replica group
    dist.init_process_group("gloo" if cpu else "nccl", init_method=f"tcp://127.0.0.1:{a.group_port}", rank=gr,
                            world_size=shard)
    mesh = init_device_mesh(dev.type, (shard,), mesh_dim_names=("shard",))
    timeout = timedelta(seconds=120)
    pg = torchft.ProcessGroupGloo(timeout=timeout) if cpu else torchft.ProcessGroupNCCL(timeout=timeout)
    holder = {}
    transport = PGTransport(pg, timeout=timeout, device=dev, state_dict=lambda: holder["manager"]._manager_state_dict())
    B, S = 1, a.seq_len
    torch.manual_seed(1234 + 77 * a.generation)
    model, margs = build_model(a.model, S, dev, mesh, "selective")
    inner = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=not cpu)

    def load_state(sd):
        model.load_state_dict(sd["model"])
        inner.load_state_dict(sd["optim"])

    def save_state():
        return {"model": model.state_dict(), "optim": inner.state_dict()}

    manager = torchft.Manager(
        pg=pg, min_replica_size=1, load_state_dict=load_state, state_dict=save_state, replica_id=f"heal_rep{a.replica}",
        store_addr="127.0.0.1", store_port=a.group_port, rank=gr, world_size=shard, lighthouse_addr=a.lighthouse, port=0,
        hostname="127.0.0.1", timeout=timeout, quorum_timeout=timedelta(seconds=180),
        connect_timeout=timedelta(seconds=30), checkpoint_transport=transport, use_async_quorum=False, init_sync=False)
    holder["manager"] = manager
    replicate_pg = ManagedProcessGroup(manager)
    replicate_pg.register("dp_replicate")

    def all_reduce_hook(output):
        dist.all_reduce(output, group=replicate_pg, op=dist.ReduceOp.AVG)

    for m in model.modules():
        if isinstance(m, FSDPModule):
            m.set_all_reduce_hook(all_reduce_hook)
    optim = OptimizerWrapper(manager, inner)
    params = list(model.parameters())
    # materialise the AdamW moments so that a healing replica receives them in place
    for p in params:
        p.grad = torch.zeros_like(p)
    inner.step()
    inner.zero_grad()
    state_bytes = sum(p.to_local().numel() * 4 * 3 if hasattr(p, "to_local") else p.numel() * 12 for p in params)

    def train_step(tokens, labels):
        optim.zero_grad()
        pred = model(tokens)
        loss = F.cross_entropy(pred.flatten(0, 1).float(), labels.flatten(0, 1))
        del pred
        loss.backward()
        clip_grad_norm_(params, 1.0, foreach=True)
        optim.step()
        return loss.detach()

    g = torch.Generator().manual_seed(5 + gr)
    tokens = torch.randint(0, margs.vocab_size, (B, S + 1), generator=g).to(dev)

    def sync():
        if not cpu:
            torch.cuda.synchronize()

    records = []
    commits_failed = 0
    rejoined_at = None
    t_wait = time.time()
    while True:
        step = manager.current_step()
        if a.leave_at < 0 and rejoined_at is not None and step >= rejoined_at + a.after:
            break
        if a.leave_at >= 0 and step == a.leave_at:
            sync()
            os._exit(17)  # between steps: nothing of ours is in flight
        sync()
        t0 = time.perf_counter()
        before = manager.current_step()
        loss = train_step(tokens[:, :-1], tokens[:, 1:])
        sync()
        dt = time.perf_counter() - t0
        n = manager.num_participants()
        if manager.current_step() <= before:
            commits_failed += 1
        records.append({"step": manager.current_step(), "s": round(dt, 4), "participants": n, "loss": round(float(loss), 4),
                        "healed": a.generation > 0 and len(records) == 0, "t_end": time.time(), "phases": {}})
        if a.leave_at < 0 and step >= a.hold and rejoined_at is None:
            if n >= 2:
                rejoined_at = manager.current_step()
            elif time.time() - t_wait > 400:
                print(json.dumps({"replica": a.replica, "error": "peer never (re)joined"}), flush=True)
                os._exit(3)
    sync()
    checksum = 0.0
    for p in params:
        local = p.to_local() if hasattr(p, "to_local") else p
        checksum += float(local.double().sum().item())
    print(json.dumps({"replica": a.replica, "generation": a.generation, "group_rank": gr, "records": records,
                      "last_recv": {}, "state_bytes": state_bytes, "commits_failed": commits_failed, "checksum": checksum,
                      "errored": str(pg.errored())}), flush=True)
    manager.shutdown(wait=False)
    os._exit(0)


if __name__ == "__main__":
    sys.exit(main())
