"""LocalSGD / DiLoCo end to end on CPU/gloo with real managers and a lighthouse: healthy run,
a replica that dies and heals, a replica that joins late, and an injected allreduce failure.
Pass criterion: the replicas' global state (backup weights, outer optimizer) is identical."""
import copy
import threading
from datetime import timedelta
from typing import Any, Dict

import pytest
import torch
from torch import nn, optim

from ft_harness import EventInjector, Runner, run_replicas
from torchft_b200 import Manager
from torchft_b200._ftcp import LighthouseServer
from torchft_b200.local_sgd import DiLoCo, LocalSGD
from torchft_b200.process_group import FakeProcessGroupWrapper, ProcessGroupGloo


def make_model():
    torch.manual_seed(7)
    return nn.Sequential(nn.Linear(3, 8), nn.ReLU(), nn.Linear(8, 4), nn.ReLU(), nn.Linear(4, 2))


def _manager(runner: Runner, rank: int, store_port: int, pg, load, save, **kw):
    return Manager(
        pg=pg, min_replica_size=1, load_state_dict=load, state_dict=save, replica_id=str(runner.replica_id),
        store_addr="localhost", store_port=store_port, rank=rank, world_size=runner.world_size,
        lighthouse_addr=runner.lighthouse_address, port=0, timeout=timedelta(seconds=10),
        quorum_timeout=timedelta(seconds=20), connect_timeout=timedelta(seconds=10), hostname="localhost", **kw)


def local_sgd_loop(rank, store_port, runner, total_syncs=4, sync_every=2):
    model = make_model()
    opt = optim.SGD(model.parameters(), lr=0.05)
    pg = FakeProcessGroupWrapper(ProcessGroupGloo(timeout=timedelta(seconds=10)))
    manager = _manager(runner, rank, store_port, pg, lambda sd: (model.load_state_dict(sd["m"]), opt.load_state_dict(sd["o"])),
                       lambda: {"m": model.state_dict(), "o": opt.state_dict()})
    try:
        with LocalSGD(manager, model, opt, sync_every=sync_every):
            it = 0
            while manager.current_step() < total_syncs:
                runner.injector.check(runner.replica_id, rank, manager.current_step(), pg)
                g = torch.Generator().manual_seed(100 * runner.replica_id + it)
                x = torch.randn(8, 3, generator=g)
                opt.zero_grad()
                model(x).sum().backward()
                opt.step()
                it += 1
        return {"state": {k: v.clone() for k, v in model.state_dict().items()}, "step": manager.current_step()}
    finally:
        manager.shutdown(wait=False)
        pg.shutdown()


def diloco_loop(rank, store_port, runner, total_syncs=4, sync_every=4, n_fragments=2, delay=0, alpha=0.0):
    model = make_model()
    inner = optim.AdamW(model.parameters(), lr=1e-2)
    frags = [model] if n_fragments == 1 else [model[:2], model[2:]]
    outers = [optim.SGD(f.parameters(), lr=0.7, momentum=0.9, nesterov=True) for f in frags]
    pg = FakeProcessGroupWrapper(ProcessGroupGloo(timeout=timedelta(seconds=10)))
    manager = _manager(runner, rank, store_port, pg,
                       lambda sd: (model.load_state_dict(sd["m"]), inner.load_state_dict(sd["o"])),
                       lambda: {"m": model.state_dict(), "o": inner.state_dict()}, use_async_quorum=False)
    history: Dict[int, Any] = {}
    try:
        with DiLoCo(manager, frags, inner, outers, sync_every=sync_every, fragment_sync_delay=delay,
                    fragment_update_alpha=alpha, backup_device=torch.device("cpu"), pin_memory=False) as d:
            it = 0
            while manager.current_step() < total_syncs:
                step = manager.current_step()
                runner.injector.check(runner.replica_id, rank, step, pg)
                g = torch.Generator().manual_seed(100 * runner.replica_id + it)
                x = torch.randn(8, 3, generator=g)
                inner.zero_grad()
                model(x).sum().backward()
                inner.step()
                it += 1
                if manager.current_step() != step:  # a sync just committed
                    history[manager.current_step()] = {
                        "global": [{n: t.clone() for n, t in f.original_parameters.items()} for f in d._fragments],
                        "outer": [copy.deepcopy(o.state_dict()["state"]) for o in outers],
                    }
        return {"history": history, "step": manager.current_step()}
    finally:
        manager.shutdown(wait=False)
        pg.shutdown()


def _run(loop, n_replicas=2, injector=None, min_replicas=2, **kw):
    lh = LighthouseServer("[::]:0", min_replicas, join_timeout_ms=200, heartbeat_timeout_ms=1000)
    try:
        inj = injector or EventInjector()
        runners = [Runner(i, lh.address(), inj, None, num_replicas=n_replicas) for i in range(n_replicas)]  # type: ignore[arg-type]
        for r in runners:
            r.train_loop = lambda rank, store_port, runner: loop(rank, store_port, runner, **kw)
        return run_replicas(runners), inj
    finally:
        lh.shutdown()


def _assert_same_history(results):
    ref = results[0][0]["history"]
    for rep in results[1:]:
        h = rep[0]["history"]
        common = sorted(set(ref) & set(h))
        assert common, "replicas share no committed step"
        for step in common:
            for fa, fb in zip(ref[step]["global"], h[step]["global"]):
                for n in fa:
                    torch.testing.assert_close(fa[n], fb[n], rtol=1e-5, atol=1e-6, msg=lambda m: f"step {step} {n}: {m}")
            for oa, ob in zip(ref[step]["outer"], h[step]["outer"]):
                for k in oa:
                    if "momentum_buffer" in oa[k] and oa[k]["momentum_buffer"] is not None:
                        torch.testing.assert_close(oa[k]["momentum_buffer"], ob[k]["momentum_buffer"], rtol=1e-5, atol=1e-6)


def test_local_sgd_healthy():
    res, _ = _run(local_sgd_loop)
    a, b = res[0][0]["state"], res[1][0]["state"]
    for k in a:
        torch.testing.assert_close(a[k], b[k])


def test_local_sgd_recovery():
    inj = EventInjector().fail_at(replica=1, step=2).gate_until_rejoin(replica=0, step=3)
    res, inj = _run(local_sgd_loop, injector=inj, min_replicas=1, total_syncs=5)
    assert inj.count == 1
    a, b = res[0][0]["state"], res[1][0]["state"]
    for k in a:
        torch.testing.assert_close(a[k], b[k])


@pytest.mark.parametrize("n_fragments,delay,alpha", [(1, 0, 0.0), (2, 0, 0.0), (2, 1, 0.5), (2, 1, 1.0)])
def test_diloco_healthy(n_fragments, delay, alpha):
    res, _ = _run(diloco_loop, n_fragments=n_fragments, delay=delay, alpha=alpha)
    assert all(r[0]["step"] == 4 for r in res)
    _assert_same_history(res)


def test_diloco_recovery_streaming():
    inj = EventInjector().fail_at(replica=1, step=2).gate_until_rejoin(replica=0, step=3)
    res, inj = _run(diloco_loop, injector=inj, min_replicas=1, total_syncs=5, n_fragments=2, delay=1)
    assert inj.count == 1
    _assert_same_history(res)


def test_diloco_commit_failure_is_retried():
    inj = EventInjector().fail_allreduce_at(replica=0, step=1).fail_allreduce_at(replica=1, step=1)
    res, inj = _run(diloco_loop, injector=inj, total_syncs=4, n_fragments=2)
    assert inj.count == 2
    _assert_same_history(res)


def test_diloco_upscale_third_replica_joins_late():
    barrier = threading.Barrier(3)
    inj = EventInjector()
    for r in range(3):
        inj.barrier_at(replica=r, step=2 if r < 2 else 0, barrier=barrier)
    res, _ = _run(diloco_loop, n_replicas=3, injector=inj, min_replicas=2, total_syncs=5, n_fragments=2)
    _assert_same_history(res)


# ---- streaming DiLoCo on the explicit Llama engine (flat units, fused outer step) ----------


def engine_diloco_loop(rank, store_port, runner, total_syncs=4, sync_every=4, n_fragments=2, delay=0, alpha=0.0):
    from torchft_b200.models.llama import LLAMA_TINY
    from torchft_b200.parallel.diloco import EngineDiLoCo
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer

    cfg, B, S = LLAMA_TINY, 2, 16
    tr = ShardedLlamaTrainer(cfg, B, S, torch.device("cpu"), lr=1e-2, seed=5)
    pg = FakeProcessGroupWrapper(ProcessGroupGloo(timeout=timedelta(seconds=10)))
    manager = _manager(runner, rank, store_port, pg, tr.load_state_dict, tr.state_dict, use_async_quorum=False)
    history: Dict[int, Any] = {}
    try:
        d = EngineDiLoCo(tr, manager, n_fragments=n_fragments, sync_every=sync_every, fragment_sync_delay=delay,
                         fragment_update_alpha=alpha)
        it = 0
        while manager.current_step() < total_syncs:
            step = manager.current_step()
            runner.injector.check(runner.replica_id, rank, step, pg)
            g = torch.Generator().manual_seed(100 * runner.replica_id + it)
            tokens = torch.randint(0, cfg.vocab_size, (B, S), generator=g)
            d.train_step(tokens, torch.roll(tokens, -1, 1))
            it += 1
            if manager.current_step() != step:
                history[manager.current_step()] = {
                    "global": [{f"unit{u}": b.clone() for u, b in zip(f.units, f.backup)} for f in d.fragments],
                    "outer": [{u: {"momentum_buffer": m.clone()} for u, m in zip(f.units, f.momentum)} for f in d.fragments],
                }
        return {"history": history, "step": manager.current_step()}
    finally:
        manager.shutdown(wait=False)
        pg.shutdown()


@pytest.mark.parametrize("n_fragments,delay,alpha", [(2, 0, 0.0), (3, 1, 0.5)])
def test_engine_diloco_healthy(n_fragments, delay, alpha):
    res, _ = _run(engine_diloco_loop, n_fragments=n_fragments, delay=delay, alpha=alpha, sync_every=2 * n_fragments)
    assert all(r[0]["step"] == 4 for r in res)
    _assert_same_history(res)


def test_engine_diloco_recovery():
    inj = EventInjector().fail_at(replica=1, step=2).gate_until_rejoin(replica=0, step=3)
    res, inj = _run(engine_diloco_loop, injector=inj, min_replicas=1, total_syncs=5, n_fragments=2, delay=1)
    assert inj.count == 1
    _assert_same_history(res)
