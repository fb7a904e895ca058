"""End-to-end fault tolerance on CPU/gloo: replica groups train a LeNet with FT-DDP; one
is killed and heals from its peer; pass criterion is identical final weights."""
import threading
from datetime import timedelta
from typing import Any, Dict

import pytest
import torch
from torch import nn, optim

from ft_harness import EventInjector, Runner, run_replicas
from torchft_b200 import DistributedDataParallel, Manager, Optimizer
from torchft_b200._ftcp import LighthouseServer
from torchft_b200.models.lenet import LeNet, synthetic_batch
from torchft_b200.process_group import FakeProcessGroupWrapper, ProcessGroupGloo


_INIT_LOCK = threading.Lock()


def ddp_train_loop(rank: int, store_port: int, runner: Runner, total_steps: int = 100, batch: int = 64,
                   use_async_quorum: bool = True, model_fn=LeNet, init_sync: bool = True) -> Dict[str, Any]:
    with _INIT_LOCK:  # replica groups are threads here: the global generator must not be shared while seeding
        torch.manual_seed(42 if not init_sync else runner.replica_id)  # init_sync must equalise different inits
        model = model_fn()
    opt = optim.SGD(model.parameters(), lr=1e-3, momentum=0.9)

    loads = []

    def load_state_dict(sd):
        loads.append(manager.current_step())
        model.load_state_dict(sd["model"])
        opt.load_state_dict(sd["optim"])

    def state_dict():
        return {"model": model.state_dict(), "optim": opt.state_dict()}

    pg = FakeProcessGroupWrapper(ProcessGroupGloo(timeout=timedelta(seconds=10)))
    manager = Manager(
        pg=pg, min_replica_size=1, load_state_dict=load_state_dict, state_dict=state_dict,
        replica_id=str(runner.replica_id), store_addr="localhost", store_port=store_port, rank=rank,
        world_size=runner.world_size, lighthouse_addr=runner.lighthouse_address, port=0,
        quorum_timeout=timedelta(seconds=20), connect_timeout=timedelta(seconds=10),
        use_async_quorum=use_async_quorum, init_sync=init_sync, hostname="localhost",
        **{"timeout": timedelta(seconds=10), **runner.manager_args},
    )
    try:
        m = DistributedDataParallel(manager, model)
        optimizer = Optimizer(manager, opt)
        crit = nn.CrossEntropyLoss()
        while manager.current_step() < total_steps:
            step = manager.current_step()
            runner.injector.check(runner.replica_id, rank, step, pg)
            x, y = synthetic_batch(batch, seed=1000 * runner.replica_id + step)
            optimizer.zero_grad()
            loss = crit(m(x), y)
            loss.backward()
            optimizer.step()
        return {"state": {k: v.clone() for k, v in model.state_dict().items()}, "step": manager.current_step(),
                "batches": manager.batches_committed(), "loads": len(loads)}
    finally:
        manager.shutdown(wait=False)
        pg.shutdown()


def _assert_same(results):
    """Rank r of every replica group must hold the same weights (each local rank forms its
    own replica-dimension communicator, so columns are compared, not whole groups)."""
    for rank in range(len(results[0])):
        ref = results[0][rank]["state"]
        for rep in results:
            for k, v in rep[rank]["state"].items():
                torch.testing.assert_close(v, ref[k], rtol=1e-5, atol=1e-6, msg=lambda m: f"rank {rank} {k}: {m}")


@pytest.mark.parametrize("use_async_quorum", [True, False])
def test_ddp_healthy(use_async_quorum):
    lh = LighthouseServer("[::]:0", 2, join_timeout_ms=100)
    try:
        inj = EventInjector()
        runners = [Runner(i, lh.address().replace("http://", "http://"), inj, ddp_train_loop,
                          train_loop_args={}, manager_args={}) for i in range(2)]
        for r in runners:
            r.train_loop = lambda rank, store_port, runner: ddp_train_loop(rank, store_port, runner, total_steps=8,
                                                                          use_async_quorum=use_async_quorum)
        res = run_replicas(runners)
        _assert_same(res)
        assert all(r[0]["step"] == 8 for r in res)
    finally:
        lh.shutdown()


@pytest.mark.parametrize("use_async_quorum", [True, False])
def test_ddp_recovery_kill_and_heal(use_async_quorum):
    """BASELINE config 1 (shortened to keep CI fast; the example script runs all 100 steps):
    replica 1 dies at step 20 of 30 and heals from replica 0."""
    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=100, heartbeat_timeout_ms=1000)
    try:
        inj = EventInjector().fail_at(replica=1, step=20).gate_until_rejoin(replica=0, step=22)
        runners = [Runner(i, lh.address(), inj, None) for i in range(2)]  # type: ignore[arg-type]
        for r in runners:
            r.train_loop = lambda rank, store_port, runner: ddp_train_loop(rank, store_port, runner, total_steps=30,
                                                                          use_async_quorum=use_async_quorum)
        res = run_replicas(runners)
        assert inj.count == 1
        _assert_same(res)
        assert all(r[0]["step"] == 30 for r in res)
    finally:
        lh.shutdown()


@pytest.mark.parametrize("init_sync", [True, False])
def test_ddp_init_sync(init_sync):
    """init_sync=True: differently initialised groups are equalised at step 0 (every group but the primary loads
    state once).  init_sync=False: the user vouches for identical initialisation, nothing is transferred."""
    lh = LighthouseServer("[::]:0", 2, join_timeout_ms=100)
    try:
        runners = [Runner(i, lh.address(), EventInjector(), None) for i in range(2)]  # type: ignore[arg-type]
        for r in runners:
            r.train_loop = lambda rank, store_port, runner: ddp_train_loop(rank, store_port, runner, total_steps=5,
                                                                          init_sync=init_sync)
        res = run_replicas(runners)
        _assert_same(res)
        assert sum(r[0]["loads"] for r in res) == (1 if init_sync else 0)
    finally:
        lh.shutdown()


def test_ddp_allreduce_failure_is_not_committed():
    lh = LighthouseServer("[::]:0", 2, join_timeout_ms=100)
    try:
        inj = EventInjector().fail_allreduce_at(replica=0, step=3)
        runners = [Runner(i, lh.address(), inj, None) for i in range(2)]  # type: ignore[arg-type]
        for r in runners:
            r.train_loop = lambda rank, store_port, runner: ddp_train_loop(rank, store_port, runner, total_steps=6)
        res = run_replicas(runners)
        assert inj.count == 1
        _assert_same(res)
    finally:
        lh.shutdown()


def test_ddp_multi_rank_groups():
    lh = LighthouseServer("[::]:0", 2, join_timeout_ms=100)
    try:
        inj = EventInjector()
        runners = [Runner(i, lh.address(), inj, None, world_size=2) for i in range(2)]  # type: ignore[arg-type]
        for r in runners:
            r.train_loop = lambda rank, store_port, runner: ddp_train_loop(rank, store_port, runner, total_steps=4)
        res = run_replicas(runners)
        _assert_same(res)
    finally:
        lh.shutdown()


def test_ddp_recovery_multi_rank_groups():
    """Groups of two ranks: rank 0 of group 1 fails, the whole group restarts (its other rank runs into the commit
    barrier's timeout), heals rank by rank from group 0 and all columns end identical
    (torchft/manager_integ_test.py test_ddp_recovery_multi_rank)."""
    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=100, heartbeat_timeout_ms=1000)
    try:
        inj = EventInjector().fail_at(replica=1, step=4, rank=0).gate_until_rejoin(replica=0, step=6)
        runners = [Runner(i, lh.address(), inj, None, world_size=2, manager_args={"timeout": timedelta(seconds=3)})  # type: ignore[arg-type]
                   for i in range(2)]
        for r in runners:
            r.train_loop = lambda rank, store_port, runner: ddp_train_loop(rank, store_port, runner, total_steps=12)
        res = run_replicas(runners)
        assert inj.count == 1
        _assert_same(res)
        assert all(r[k]["step"] == 12 for r in res for k in range(2))
    finally:
        lh.shutdown()


def test_quorum_timeout_is_prompt():
    import time
    from torch.distributed import TCPStore

    lh = LighthouseServer("[::]:0", 2, join_timeout_ms=100)  # needs 2 replicas, only one shows up
    store = TCPStore(host_name="localhost", port=0, is_master=True, wait_for_workers=False)
    pg = ProcessGroupGloo()
    manager = Manager(pg=pg, min_replica_size=2, load_state_dict=lambda x: None, state_dict=lambda: None,
                      store_addr="localhost", store_port=store.port, rank=0, world_size=1,
                      lighthouse_addr=lh.address(), port=0, use_async_quorum=False, hostname="localhost",
                      timeout=timedelta(seconds=5), connect_timeout=timedelta(seconds=5))
    try:
        t0 = time.time()
        with pytest.raises(TimeoutError):
            manager.start_quorum(timeout=timedelta(milliseconds=100))
        assert time.time() - t0 < 2.0
    finally:
        manager.shutdown(wait=False)
        lh.shutdown()
