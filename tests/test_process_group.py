"""Process-group conformance: every collective on world-size-1 groups, numeric checks on
multi-rank gloo groups (ranks are threads sharing one store), reconfiguration, and the
resiliency contract (a peer that goes away makes the survivors' collectives fail fast)."""
import os
import time
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
from torch.distributed.distributed_c10d import (AllgatherOptions, AllreduceOptions, AllToAllOptions, BarrierOptions,
                                                BroadcastOptions, ReduceOp, ReduceScatterOptions)

from torchft_b200.process_group import (
    ErrorSwallowingProcessGroupWrapper,
    FakeProcessGroupWrapper,
    ManagedProcessGroup,
    ProcessGroup,
    ProcessGroupBabyGloo,
    ProcessGroupDummy,
    ProcessGroupGloo,
    create_store_client,
)
from torchft_b200.work import _DummyWork


def _exercise_all_collectives(pg, skip=()):
    """Shapes and dtypes survive every collective on a group of one."""
    t = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    ops = {
        "allreduce": lambda: pg.allreduce([t.clone()], AllreduceOptions()),
        "allreduce_coalesced": lambda: pg.allreduce_coalesced([t.clone(), t.clone()]),
        "allgather": lambda: pg.allgather([[torch.empty_like(t)]], [t.clone()], AllgatherOptions()),
        "allgather_into_tensor_coalesced": lambda: pg.allgather_into_tensor_coalesced([torch.empty_like(t)], [t.clone()], AllgatherOptions()),
        "alltoall_base": lambda: pg.alltoall_base(torch.empty_like(t), t.clone(), [], [], AllToAllOptions()),
        "barrier": lambda: pg.barrier(BarrierOptions()),
        "broadcast": lambda: pg.broadcast([t.clone()], BroadcastOptions()),
        "broadcast_one": lambda: pg.broadcast_one(t.clone(), 0),
        "reduce_scatter": lambda: pg.reduce_scatter([torch.empty_like(t)], [[t.clone()]], ReduceScatterOptions()),
        "reduce_scatter_tensor_coalesced": lambda: pg.reduce_scatter_tensor_coalesced([torch.empty_like(t)], [t.clone()], ReduceScatterOptions()),
    }
    for name, fn in ops.items():
        if name in skip:
            with pytest.raises(RuntimeError):
                fn()
            continue
        w = fn()
        w.wait()
        w.get_future().wait()


def _store():
    return dist.TCPStore("localhost", 0, is_master=True, wait_for_workers=False)


def test_dummy_pg():
    pg = ProcessGroupDummy(0, 1)
    _exercise_all_collectives(pg)
    pg.configure("x", "r", 0, 1)
    assert pg.configure_count == 1 and pg.size() == 1


def test_gloo_world1_all_collectives_and_timeouts():
    store = _store()
    pg = ProcessGroupGloo(timeout=timedelta(seconds=10))
    pg.configure(f"localhost:{store.port}/a", "r", 0, 1)
    _exercise_all_collectives(pg, skip=("reduce_scatter", "reduce_scatter_tensor_coalesced"))
    pg.set_timeout(timedelta(seconds=3))
    assert pg._timeout == timedelta(seconds=3)
    # a second configure needs (and gets) a fresh prefix
    pg.configure(f"localhost:{store.port}/b", "r", 0, 1)
    pg.allreduce([torch.ones(2)], ReduceOp.SUM).wait()
    pg.shutdown()


def _multi(world, cls=ProcessGroupGloo, prefix="m"):
    store = _store()
    pgs = [cls(timeout=timedelta(seconds=10)) for _ in range(world)]
    with ThreadPoolExecutor(max_workers=world) as ex:
        list(ex.map(lambda r: pgs[r].configure(f"localhost:{store.port}/{prefix}", "rep", r, world), range(world)))
    return store, pgs


def _run(pgs, fn):
    with ThreadPoolExecutor(max_workers=len(pgs)) as ex:
        return list(ex.map(lambda r: fn(r, pgs[r]), range(len(pgs))))


def test_gloo_multi_rank_numerics():
    world = 3
    store, pgs = _multi(world)
    try:
        def allreduce(r, pg):
            t = torch.full((4,), float(r + 1))
            pg.allreduce([t], ReduceOp.SUM).wait()
            return t
        for t in _run(pgs, allreduce):
            assert torch.equal(t, torch.full((4,), 6.0))

        def allgather(r, pg):
            outs = [[torch.zeros(2) for _ in range(world)]]
            pg.allgather(outs, [torch.full((2,), float(r))], AllgatherOptions()).wait()
            return outs[0]
        for outs in _run(pgs, allgather):
            assert [o[0].item() for o in outs] == [0.0, 1.0, 2.0]

        def bcast(r, pg):
            t = torch.full((3,), float(r))
            pg.broadcast_one(t, 1).wait()
            return t
        assert all(torch.equal(t, torch.ones(3)) for t in _run(pgs, bcast))

        def a2a(r, pg):
            out = torch.zeros(world)
            pg.alltoall_base(out, torch.full((world,), float(r)), [], [], AllToAllOptions()).wait()
            return out
        for out in _run(pgs, a2a):
            assert out.tolist() == [0.0, 1.0, 2.0]

        def sendrecv(r, pg):
            if r == 0:
                pg.send([torch.tensor([42.0])], 1, 7).wait()
                return None
            if r == 1:
                t = torch.zeros(1)
                pg.recv([t], 0, 7).wait()
                return t.item()
        assert _run(pgs, sendrecv)[1] == 42.0
        _run(pgs, lambda r, pg: pg.barrier().wait())
    finally:
        for pg in pgs:
            pg.shutdown()


@pytest.mark.parametrize("cls", [ProcessGroupGloo, ProcessGroupBabyGloo])
def test_gloo_resiliency_peer_leaves(cls):
    """After one rank shuts down, the survivors' next collective must raise within the
    timeout instead of hanging (in-process and subprocess-backed groups alike)."""
    world = 2
    store = _store()
    # a subprocess-backed group needs its timeout for starting the child interpreter as well
    pgs = [cls(timeout=timedelta(seconds=1 if cls is ProcessGroupGloo else 30)) for _ in range(world)]
    with ThreadPoolExecutor(max_workers=world) as ex:
        list(ex.map(lambda r: pgs[r].configure(f"localhost:{store.port}/res", "rep", r, world), range(world)))
    _run(pgs, lambda r, pg: pg.allreduce([torch.ones(1)], ReduceOp.SUM).wait())
    pgs[1].shutdown()
    t0 = time.time()
    with pytest.raises(Exception):
        pgs[0].allreduce([torch.ones(1)], ReduceOp.SUM).wait(timedelta(seconds=5))
    assert time.time() - t0 < 15
    # and it can be reconfigured alone afterwards
    pgs[0].configure(f"localhost:{store.port}/res2", "rep", 0, 1)
    pgs[0].allreduce([torch.ones(1)], ReduceOp.SUM).wait()
    pgs[0].shutdown()


def test_error_swallowing_and_fake_wrappers():
    inner = ProcessGroupDummy(0, 1)
    fake = FakeProcessGroupWrapper(inner)
    fake.configure("addr", "r", 0, 1)
    t = torch.ones(2)
    fake.allreduce([t], ReduceOp.SUM).wait()
    fake.report_future_error(RuntimeError("injected"))
    w = fake.allreduce([t], ReduceOp.SUM)
    with pytest.raises(RuntimeError, match="injected"):
        w.get_future().wait()
    fake.allreduce([t], ReduceOp.SUM).get_future().wait()  # only the next one fails
    fake.report_error(RuntimeError("latched"))
    assert "latched" in str(fake.errored())
    fake.configure("addr2", "r", 0, 1)
    assert fake.errored() is None

    sw = ErrorSwallowingProcessGroupWrapper(FakeProcessGroupWrapper(ProcessGroupDummy(0, 1)))
    sw.configure("a", "r", 0, 1)
    sw._pg.report_future_error(RuntimeError("boom"))
    w = sw.allreduce([t], ReduceOp.SUM)
    w.get_future().wait()
    w.wait()
    assert "boom" in str(sw.error())
    assert isinstance(sw.allreduce([t], ReduceOp.SUM), _DummyWork)  # no-op until reconfigured
    sw.configure("b", "r", 0, 1)
    assert sw.error() is None


def test_managed_process_group():
    from unittest.mock import MagicMock

    manager = MagicMock()
    manager._pg = ProcessGroupDummy(0, 1)
    manager.num_participants.return_value = 123
    manager.allreduce.return_value = _DummyWork(None)
    pg = ManagedProcessGroup(manager)
    assert pg.size() == 123
    t = torch.zeros(3)
    pg.allreduce([t], ReduceOp.SUM).wait()
    assert manager.allreduce.call_count == 1
    assert manager.allreduce.call_args.kwargs["reduce_op"] == ReduceOp.SUM


def test_baby_gloo_reconfigure_and_active_work():
    world = 2
    store = _store()
    pgs = [ProcessGroupBabyGloo(timeout=timedelta(seconds=20)) for _ in range(world)]
    try:
        with ThreadPoolExecutor(max_workers=world) as ex:
            list(ex.map(lambda r: pgs[r].configure(f"localhost:{store.port}/baby1", "rep", r, world), range(world)))

        def allreduce(r, pg):
            t = torch.full((4,), float(r + 1))
            pg.allreduce([t], ReduceOp.SUM).wait()
            return t
        for t in _run(pgs, allreduce):
            assert torch.equal(t, torch.full((4,), 3.0))
        assert pgs[0].num_active_work() == 0
        old = pgs[0]._proc
        with ThreadPoolExecutor(max_workers=world) as ex:
            list(ex.map(lambda r: pgs[r].configure(f"localhost:{store.port}/baby2", "rep", r, world), range(world)))
        assert not old.is_alive()  # the previous worker process is gone
        for t in _run(pgs, allreduce):
            assert torch.equal(t, torch.full((4,), 3.0))
        with pytest.raises(RuntimeError):
            pgs[0].reduce_scatter([torch.zeros(1)], [[torch.zeros(1)]])
    finally:
        for pg in pgs:
            pg.shutdown()


def test_create_store_client_and_base_class_contract():
    store = _store()
    c = create_store_client(f"localhost:{store.port}/some/prefix", timedelta(seconds=5))
    c.set("k", "v")
    assert c.get("k") == b"v"
    base = ProcessGroup(0, 1)
    with pytest.raises(NotImplementedError):
        base.allreduce([torch.zeros(1)])
    with pytest.raises(NotImplementedError):
        base.configure("a", "b", 0, 1)
    assert base.errored() is None
    with pytest.raises(ValueError):
        base.group_name
    base._set_group_name("x")
    assert base.group_name == "x"


def test_registered_pg_serves_functional_collectives_and_device_mesh():
    """A registered process group resolves for torch's functional collectives and DeviceMesh.from_group
    (torchft/process_group_test.py:732-774).  Runs in a child: it initialises torch.distributed."""
    import subprocess
    import sys

    child = r'''
import sys, torch, torch.distributed as dist
from datetime import timedelta
from torch.distributed import TCPStore
from torch.distributed import _functional_collectives as fc
from torch.distributed.device_mesh import DeviceMesh
from torchft_b200.process_group import ProcessGroupGloo
store = TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
dist.init_process_group("gloo", store=dist.PrefixStore("default", store), rank=0, world_size=1)
pg = ProcessGroupGloo(timeout=timedelta(seconds=10))
pg.configure(f"127.0.0.1:{store.port}/ft", "rep0", 0, 1)
pg.register("ftb200_functional")
t = torch.arange(10, dtype=torch.float32)
out = fc.wait_tensor(fc.all_reduce(t, "sum", pg))
assert torch.equal(out, t)
mesh = DeviceMesh.from_group(pg, "cpu")
assert mesh.size() == 1 and mesh.get_group() is not None
pg.unregister()
print("ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", child], capture_output=True, text=True, timeout=120,
                       env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


def test_baby_gloo_on_thread_backed_context(monkeypatch):
    """The subprocess-backed group runs unchanged with its worker on a thread (DummyContext): two ranks in
    one interpreter, allreduce, reconfigure, an injected worker death."""
    from torchft_b200.multiprocessing_dummy_context import DummyContext, ThreadProcess

    monkeypatch.setattr(ProcessGroupBabyGloo, "_mp_context", staticmethod(DummyContext))
    world = 2
    store = _store()
    pgs = [ProcessGroupBabyGloo(timeout=timedelta(seconds=20)) for _ in range(world)]
    try:
        for gen in ("a", "b"):
            with ThreadPoolExecutor(max_workers=world) as ex:
                list(ex.map(lambda r: pgs[r].configure(f"localhost:{store.port}/thr{gen}", "rep", r, world), range(world)))
            assert all(isinstance(pg._proc, ThreadProcess) for pg in pgs)

            def allreduce(r, pg):
                t = torch.full((4,), float(r + 1))
                pg.allreduce([t], ReduceOp.SUM).wait()
                return t
            for t in _run(pgs, allreduce):
                assert torch.equal(t, torch.full((4,), 3.0))
            assert pgs[0].num_active_work() == 0
        # the worker "dies": outstanding and later work fails instead of hanging
        proc = pgs[1]._proc
        proc.kill()
        proc.join(5)
        assert not proc.is_alive()
        with pytest.raises(Exception):
            pgs[1].allreduce([torch.ones(1)], ReduceOp.SUM).wait(timedelta(seconds=5))
    finally:
        for pg in pgs:
            pg.shutdown()


@pytest.mark.parametrize("cls", [ProcessGroupGloo, ProcessGroupBabyGloo])
def test_configure_times_out_when_peers_never_arrive(cls):
    """configure() for a world of two with nobody else joining gives up after the group's timeout instead of hanging
    (torchft/process_group_test.py test_gloo_timeout / test_baby_gloo_timeout)."""
    store = _store()
    # the subprocess-backed group also needs time to start its child, so it gets a longer timeout
    secs = 0.5 if cls is ProcessGroupGloo else 12.0
    pg = cls(timeout=timedelta(seconds=secs))
    t0 = time.time()
    with pytest.raises(Exception):
        pg.configure(f"localhost:{store.port}/lonely", "rep", 0, 2)
    assert time.time() - t0 < secs + 20
    pg.shutdown()
