"""Manager state machine against a mocked control-plane client and process group.
The cases follow the behaviours torchft/manager_test.py pins down."""
import threading
import time
from datetime import timedelta
from unittest.mock import MagicMock, create_autospec, patch

import pytest
import torch
from torch.distributed import ReduceOp, TCPStore

from torchft_b200._ftcp import QuorumResult
from torchft_b200.checkpointing.transport import CheckpointTransport
from torchft_b200.manager import MANAGER_ADDR_KEY, REPLICA_ID_KEY, Manager, WorldSizeMode
from torchft_b200.process_group import ProcessGroup
from torchft_b200.work import _DummyWork


def quorum(**kw):
    q = QuorumResult()
    q.quorum_id = 123
    q.replica_rank = 1
    q.replica_world_size = 2
    q.recover_src_manager_address = "manager address"
    q.store_address = "localhost:1/prefix"
    q.max_step = 1
    q.max_replica_rank = 1
    q.max_world_size = 2
    q.heal = False
    for k, v in kw.items():
        setattr(q, k, v)
    return q


class Harness:
    def __init__(self, **mgr_kw):
        self.store = TCPStore("localhost", 0, is_master=True, wait_for_workers=False)
        self.store.set(MANAGER_ADDR_KEY, "dummy")
        self.store.set(REPLICA_ID_KEY, "dummy_id")
        self.pg = create_autospec(ProcessGroup, instance=True)
        self.pg.errored.return_value = None
        self.pg.allreduce.side_effect = lambda tensors, opts=None, **kw: _DummyWork(tensors)
        self.transport = create_autospec(CheckpointTransport, instance=True)
        self.transport.metadata.return_value = "meta"
        self.loaded = []
        self.patcher = patch("torchft_b200.manager.ManagerClient", autospec=True)
        self.client_cls = self.patcher.start()
        kw = dict(pg=self.pg, min_replica_size=2, load_state_dict=self.loaded.append, state_dict=lambda: {"w": 1},
                  store_addr="localhost", store_port=self.store.port, rank=1, world_size=2,
                  checkpoint_transport=self.transport, timeout=timedelta(seconds=10))
        kw.update(mgr_kw)
        self.manager = Manager(**kw)
        self.client = self.manager._client

    def close(self):
        self.manager.shutdown(wait=False)
        self.patcher.stop()


@pytest.fixture
def h():
    x = Harness()
    yield x
    x.close()


def test_state_dict_roundtrip(h):
    assert h.manager.state_dict() == {"step": 0, "batches_committed": 0}
    h.manager.load_state_dict({"step": 1234, "batches_committed": 2345})
    assert h.manager.current_step() == 1234 and h.manager.batches_committed() == 2345


def test_user_state_dict_registry(h):
    assert h.manager._manager_state_dict() == {"user": {"default": {"w": 1}}, "torchft": {"step": 0, "batches_committed": 0}}
    h.manager.register_state_dict_fn("extra", lambda sd: None, lambda: "x")
    assert h.manager._manager_state_dict()["user"]["extra"] == "x"
    with pytest.raises(AssertionError):
        h.manager.register_state_dict_fn("extra", lambda sd: None, lambda: "y")


def test_quorum_happy_path_and_commit(h):
    h.client._quorum.return_value = quorum()
    h.client.should_commit.return_value = True
    m = h.manager
    assert m._quorum_id == -1 and m.current_step() == 0
    m.start_quorum()
    t = torch.tensor([2.0, 4.0])
    m.allreduce(t).wait()
    assert torch.equal(t, torch.tensor([1.0, 2.0]))  # averaged over 2 participants
    assert m.should_commit()
    assert m._quorum_id == 123 and m.current_step() == 1 and m.batches_committed() == 2
    assert h.pg.configure.call_count == 1
    assert h.pg.configure.call_args.args[0] == "localhost:1/prefix/torchft/123/1"
    assert h.pg.configure.call_args.args[2:] == (1, 2)
    # unchanged quorum id: no reconfigure
    m.start_quorum()
    m.should_commit()
    assert h.pg.configure.call_count == 1
    assert h.client._quorum.call_args.kwargs["step"] == 1 or h.client._quorum.call_args_list[0].kwargs["step"] == 0


def test_heal_sync_applies_state_before_step():
    h = Harness(use_async_quorum=False)
    try:
        h.client._quorum.return_value = quorum(heal=True, max_step=20, recover_src_replica_rank=0, max_replica_rank=None,
                                               max_world_size=1)
        h.client._checkpoint_metadata.return_value = "src_meta"
        h.client.should_commit.return_value = True
        h.transport.recv_checkpoint.return_value = {"user": {"default": {"w": 7}}, "torchft": {"step": 20, "batches_committed": 40}}
        m = h.manager
        m.start_quorum()
        assert h.loaded == [{"w": 7}] and m.current_step() == 20 and not m._healing
        assert h.transport.recv_checkpoint.call_args.kwargs["metadata"] == "src_meta"
        # synchronous quorum: everybody is healthy, both replicas participate
        assert m.num_participants() == 2 and m.is_participating()
        assert m.should_commit() and m.current_step() == 21
    finally:
        h.close()


def test_heal_async_contributes_zeros_then_applies(h):
    h.client._quorum.return_value = quorum(heal=True, max_step=20, recover_src_replica_rank=0, max_replica_rank=None,
                                           max_world_size=1)
    h.client._checkpoint_metadata.return_value = "src_meta"
    h.client.should_commit.return_value = True
    h.transport.recv_checkpoint.return_value = {"user": {"default": {"w": 9}}, "torchft": {"step": 20, "batches_committed": 40}}
    m = h.manager
    m.start_quorum()
    m.wait_quorum()
    assert m._healing and not m.is_participating() and m.num_participants() == 1
    t = torch.ones(3)
    m.allreduce(t).wait()
    assert torch.equal(t, torch.zeros(3))  # a healing replica contributes nothing
    assert h.loaded == []  # user state is applied from the main thread, at commit time
    h.manager._min_replica_size = 1
    assert m.should_commit()
    assert h.loaded == [{"w": 9}] and m.current_step() == 21


def test_send_checkpoint_to_recovering_peers(h):
    h.client._quorum.return_value = quorum(recover_dst_replica_ranks=[0], max_step=5)
    h.client.should_commit.return_value = True
    h.manager.start_quorum()
    h.manager.wait_quorum()
    kw = h.transport.send_checkpoint.call_args.kwargs
    assert kw["dst_ranks"] == [0] and kw["step"] == 5 and kw["state_dict"]["user"] == {"default": {"w": 1}}


def test_allreduce_error_latches_and_blocks_commit(h):
    h.client._quorum.return_value = quorum()
    h.client.should_commit.side_effect = lambda rank, step, vote, timeout: vote
    m = h.manager
    m.start_quorum()
    h.pg.allreduce.side_effect = RuntimeError("nccl blew up")
    t = torch.ones(2)
    w = m.allreduce(t)
    assert isinstance(w, _DummyWork) and m.errored() is not None
    h.pg.allreduce.side_effect = lambda tensors, opts=None, **kw: _DummyWork(tensors)
    assert isinstance(m.allreduce(t), _DummyWork)  # no-op for the rest of the step
    assert not m.should_commit() and m.current_step() == 0
    assert h.client.should_commit.call_args.args[2] is False
    m.start_quorum()  # clears the latch
    assert m.errored() is None
    assert m.should_commit() and m.current_step() == 1


def test_future_error_and_pg_errored(h):
    h.client._quorum.return_value = quorum()
    h.client.should_commit.side_effect = lambda rank, step, vote, timeout: vote
    m = h.manager
    m.start_quorum()
    bad = torch.futures.Future()
    bad.set_exception(RuntimeError("late failure"))
    work = MagicMock()
    work.get_future.return_value = bad
    h.pg.allreduce.side_effect = lambda tensors, opts=None, **kw: work
    m.allreduce(torch.ones(1)).wait()
    assert m.errored() is not None
    m.start_quorum()
    h.pg.allreduce.side_effect = lambda tensors, opts=None, **kw: _DummyWork(tensors)
    h.pg.errored.return_value = RuntimeError("aborted")
    assert not m.should_commit()


def test_fixed_with_spares():
    h = Harness(world_size_mode=WorldSizeMode.FIXED_WITH_SPARES, min_replica_size=2)
    try:
        h.client._quorum.return_value = quorum(replica_rank=2, replica_world_size=3, max_replica_rank=2, max_world_size=3)
        h.client.should_commit.return_value = True
        m = h.manager
        m.start_quorum()
        assert m.num_participants() == 2 and m.participating_rank() is None and not m.is_participating()
        t = torch.ones(2)
        m.allreduce(t).wait()
        assert torch.equal(t, torch.zeros(2))
        assert m.should_commit() and m.batches_committed() == 2
    finally:
        h.close()


def test_allow_heal_false(h):
    h.client._quorum.return_value = quorum(heal=True, max_step=20, recover_src_replica_rank=0)
    h.manager.start_quorum(allow_heal=False)
    h.manager.wait_quorum()
    assert not h.manager._healing and h.transport.recv_checkpoint.call_count == 0


@pytest.mark.parametrize("op,expect", [(ReduceOp.AVG, 1.0), (ReduceOp.SUM, 2.0), (ReduceOp.MAX, 2.0)])
def test_allreduce_numerics_per_op(h, op, expect):
    h.client._quorum.return_value = quorum()
    h.manager.start_quorum()
    t = torch.tensor([2.0])
    h.manager.allreduce(t, reduce_op=op).wait()
    assert t.item() == expect
    with pytest.raises(ValueError):
        h.manager.allreduce(torch.tensor([1]), reduce_op=ReduceOp.AVG)


def test_wrap_future_timeout_and_default(h):
    fut = torch.futures.Future()
    wrapped = h.manager.wrap_future(fut, default=2, timeout=timedelta(seconds=0.05))
    assert wrapped.wait() == 2 and h.manager.errored() is not None
    h.manager._errored = None
    ok = torch.futures.Future()
    w2 = h.manager.wrap_future(ok, default=-1)
    ok.set_result(5)
    assert w2.wait() == 5 and h.manager.errored() is None


def test_max_retries():
    h = Harness(max_retries=2)
    try:
        h.client._quorum.return_value = quorum()
        h.client.should_commit.return_value = False
        m = h.manager
        for _ in range(2):
            m.start_quorum()
            assert not m.should_commit()
        m.start_quorum()
        with pytest.raises(RuntimeError, match="exceeding max_retries=2"):
            m.should_commit()
        assert h.client._quorum.call_args.kwargs["commit_failures"] == 2
    finally:
        h.close()


def test_timeouts_and_flags_plumbed():
    h = Harness(init_sync=False, quorum_timeout=timedelta(seconds=7))
    try:
        h.client._quorum.return_value = quorum()
        h.client.should_commit.return_value = True
        h.manager.start_quorum(shrink_only=True, timeout=timedelta(seconds=12))
        h.manager.wait_quorum()
        kw = h.client._quorum.call_args.kwargs
        assert kw["timeout"] == timedelta(seconds=12) and kw["shrink_only"] is True and kw["init_sync"] is False
        h.manager.should_commit(timeout=timedelta(seconds=23))
        assert h.client.should_commit.call_args.kwargs["timeout"] == timedelta(seconds=23)
    finally:
        h.close()


def test_env_timeout_override(monkeypatch):
    monkeypatch.setenv("TORCHFT_TIMEOUT_SEC", "3")
    monkeypatch.setenv("TORCHFT_QUORUM_RETRIES", "4")
    h = Harness()
    try:
        assert h.manager._timeout == timedelta(seconds=3) and h.manager._quorum_retries == 4
    finally:
        h.close()


def test_pg_configure_failure_is_reported(h):
    h.client._quorum.return_value = quorum()
    h.client.should_commit.side_effect = lambda rank, step, vote, timeout: vote
    h.pg.configure.side_effect = RuntimeError("no route to peer")
    h.manager.start_quorum()
    h.manager.wait_quorum()
    assert h.manager.errored() is not None
    assert not h.manager.should_commit()


def test_state_dict_read_lock(h):
    m = h.manager
    m.disallow_state_dict_read()
    m.disallow_state_dict_read()  # idempotent
    got = []
    t = threading.Thread(target=lambda: got.append(m._manager_state_dict()))
    t.start()
    time.sleep(0.1)
    assert got == []
    m.allow_state_dict_read()
    t.join(5)
    assert len(got) == 1


def test_managed_future_callbacks_run_in_order_after_normalisation(h):
    """Callbacks chained on the work's future see the averaged tensor and run in the order
    they were added, only once the work is waited on."""
    h.client._quorum.return_value = quorum()
    h.manager.start_quorum()
    t = torch.tensor([4.0])
    order = []
    work = h.manager.allreduce(t)  # AVG over 2 participants
    fut = work.get_future()

    def first(f):
        order.append(("first", float(f.value().item() if isinstance(f.value(), torch.Tensor) else f.value()[0].item())))
        return f.value()

    def second(f):
        order.append(("second", None))
        return f.value()

    fut.then(first).then(second)
    assert order == []  # nothing runs before the wait
    work.wait()
    fut.wait()
    assert [name for name, _ in order] == ["first", "second"]
    assert order[0][1] == 2.0 and t.item() == 2.0


def test_allreduce_delta_falls_back_to_subtract_then_allreduce(h):
    h.client._quorum.return_value = quorum()
    h.manager.start_quorum()
    a, b, out = torch.tensor([5.0, 3.0]), torch.tensor([1.0, 1.0]), torch.zeros(2)
    h.manager.allreduce_delta(out, a, b, should_quantize=False).wait()
    torch.testing.assert_close(out, torch.tensor([2.0, 1.0]))  # (a - b) / 2 participants
    assert h.pg.allreduce.call_count == 1


def test_heal_async_not_enough_participants(h):
    """A healing replica does not count: with only one up-to-date replica and min_replica_size 2 the step must not
    commit, although this replica still receives its state (torchft/manager_test.py test_quorum_heal_async_not_enough_participants)."""
    h.client._quorum.return_value = quorum(heal=True, max_step=20, recover_src_replica_rank=0, max_replica_rank=None,
                                           max_world_size=1)
    h.client._checkpoint_metadata.return_value = "src_meta"
    h.client.should_commit.side_effect = lambda rank, step, vote, timeout: vote
    h.transport.recv_checkpoint.return_value = {"user": {"default": {"w": 9}}, "torchft": {"step": 20, "batches_committed": 40}}
    m = h.manager
    m.start_quorum()
    m.wait_quorum()
    assert m.num_participants() == 1 and not m.is_participating()
    m.allreduce(torch.ones(2)).wait()
    assert not m.should_commit()  # 1 participant < min_replica_size 2
    assert h.client.should_commit.call_args.args[2] is False or h.client.should_commit.call_args.kwargs.get("should_commit") is False
    assert h.loaded == [{"w": 9}]  # the fetched state is applied all the same
    assert m.current_step() == 20  # healed to the peers' step, nothing committed on top


def test_checkpoint_errors_are_latched_not_raised(h):
    """A failing state transfer (fetching as well as serving) ends in the error latch and a step that does not commit."""
    h.client.should_commit.side_effect = lambda rank, step, vote, timeout: vote
    m = h.manager
    # fetching
    h.client._quorum.return_value = quorum(heal=True, max_step=20, recover_src_replica_rank=0, max_replica_rank=None,
                                           max_world_size=1)
    h.client._checkpoint_metadata.return_value = "src_meta"
    h.transport.recv_checkpoint.side_effect = RuntimeError("peer went away")
    m.start_quorum()
    m.wait_quorum()
    assert "peer went away" in str(m.errored())
    assert not m.should_commit() and h.loaded == []
    # serving
    h.transport.recv_checkpoint.side_effect = None
    h.transport.send_checkpoint.side_effect = RuntimeError("disk on fire")
    h.client._quorum.return_value = quorum(recover_dst_replica_ranks=[0], max_step=5)
    m.start_quorum()
    m.wait_quorum()
    assert "disk on fire" in str(m.errored())
    assert not m.should_commit()
    # the latch is cleared by the next quorum
    h.transport.send_checkpoint.side_effect = None
    h.client._quorum.return_value = quorum()
    m.start_quorum()
    m.wait_quorum()
    assert m.errored() is None


def test_state_dict_lock_concurrent_readers_and_writer(h):
    """Readers of the state (healing peers) and the writer (the optimizer step) exclude each other; readers run
    concurrently with each other."""
    m = h.manager
    order = []
    barrier = threading.Barrier(3)

    def reader(i):
        barrier.wait(5)
        sd = m._manager_state_dict()
        order.append(("read", i, sd["user"]["default"]))

    ts = [threading.Thread(target=reader, args=(i,)) for i in range(2)]
    m.disallow_state_dict_read()  # the optimizer is about to mutate the weights
    for t in ts:
        t.start()
    barrier.wait(5)
    time.sleep(0.2)
    assert order == []  # both readers are held back
    order.append(("write",))
    m.allow_state_dict_read()
    for t in ts:
        t.join(5)
    assert order[0] == ("write",) and sorted(o[1] for o in order[1:]) == [0, 1]


def test_managed_future_chain_may_change_types_and_failures_are_latched(h):
    """Each callback receives what the previous one returned (tensor -> float -> str); a callback that raises does
    not raise out of wait(): the error is latched and the future resolves to the default
    (torchft/_test/managed_work_test.py test_callbacks_changing_return_types)."""
    h.client._quorum.return_value = quorum()
    h.client.should_commit.side_effect = lambda rank, step, vote, timeout: vote
    m = h.manager
    m.start_quorum()
    t = torch.tensor([6.0])
    work = m.allreduce(t)
    seen = []
    fut = work.get_future().then(lambda f: float(f.value()[0].item() if not isinstance(f.value(), torch.Tensor) else f.value().item()))
    fut = fut.then(lambda f: seen.append(f.value()) or f"value={f.value()}")
    fut = fut.then(lambda f: seen.append(f.value()) or len(f.value()))
    assert seen == []
    work.wait()
    assert fut.wait() == len("value=3.0") and seen == [3.0, "value=3.0"]
    assert m.errored() is None

    work = m.allreduce(torch.tensor([1.0]))

    def boom(f):
        raise ValueError("callback failed")

    fut = work.get_future().then(boom)
    work.wait()
    fut.wait()  # does not raise
    assert "callback failed" in str(m.errored())
    assert not m.should_commit()


def test_unreachable_store_fails_within_connect_timeout():
    import socket as _socket

    with _socket.socket() as s:  # a port nobody listens on
        s.bind(("127.0.0.1", 0))
        dead_port = s.getsockname()[1]
    pg = create_autospec(ProcessGroup, instance=True)
    t0 = time.monotonic()
    with pytest.raises(Exception):
        Manager(pg=pg, min_replica_size=1, load_state_dict=None, state_dict=None, store_addr="127.0.0.1", store_port=dead_port,
                rank=1, world_size=2, connect_timeout=timedelta(seconds=2), timeout=timedelta(seconds=5))
    assert time.monotonic() - t0 < 30


class _CudaLike(torch.Tensor):
    """A CPU tensor that says it lives on a GPU: takes the manager down its CUDA-only branches without one."""
    is_cuda = property(lambda self: True)


def test_quantized_allreduce_is_averaged_on_a_group_that_fuses_the_scale(h):
    """A group that can fold 1/participants into its unquantised allreduce (``supports_fused_scale``) does not do
    so for the quantised collective, which reduces with SUM: the manager has to divide."""
    h.pg.supports_fused_scale = True
    h.client._quorum.return_value = quorum()
    h.manager.start_quorum()
    x = torch.full((256,), 6.0).as_subclass(_CudaLike)
    with patch("torch.cuda.current_stream", return_value=None), \
            patch("torchft_b200.collectives.allreduce_quantized",
                  side_effect=lambda tensors, op, pg, stream=None: _DummyWork(tensors)) as q:
        h.manager.allreduce(x, should_quantize=True).wait()
    assert q.call_count == 1 and q.call_args[0][1] == ReduceOp.SUM
    assert torch.allclose(x.as_subclass(torch.Tensor), torch.full((256,), 3.0))  # two participants
    # the unquantised path of the same group passes the scale down instead
    h.pg.allreduce = MagicMock(side_effect=lambda tensors, op=None, **kw: _DummyWork(tensors))
    y = torch.full((256,), 6.0)
    h.manager.allreduce(y).wait()
    assert h.pg.allreduce.call_args.kwargs["scale"] == 0.5
    assert torch.allclose(y, torch.full((256,), 6.0)) and h.manager.errored() is None
