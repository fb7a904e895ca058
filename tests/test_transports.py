"""Checkpoint transport contract: 1->2 fan-out, 1->1, then a tiny timeout must raise."""
import threading
import time
import urllib.error
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist

from torchft_b200.checkpointing.http_transport import HTTPTransport
from torchft_b200.checkpointing.pg_transport import PGTransport
from torchft_b200.process_group import ProcessGroupGloo


def make_state(seed):
    g = torch.Generator().manual_seed(seed)
    return {"rng": torch.rand(2, 3, generator=g), "nested": {"w": torch.arange(10, dtype=torch.float32), "i": torch.tensor([1, 2])},
            "str": "foo", "int": 1234, "list": [1.5, torch.ones(3, dtype=torch.bfloat16)]}


def assert_state_equal(a, b):
    assert a["str"] == b["str"] and a["int"] == b["int"]
    torch.testing.assert_close(a["rng"], b["rng"])
    torch.testing.assert_close(a["nested"]["w"], b["nested"]["w"])
    torch.testing.assert_close(a["nested"]["i"], b["nested"]["i"])
    assert a["list"][0] == b["list"][0]
    torch.testing.assert_close(a["list"][1], b["list"][1])


def run_multi_recovery(init_transport, world=3):
    barrier = threading.Barrier(world)
    timeout = timedelta(seconds=10)
    want = make_state(0)

    def run(rank):
        transport = init_transport(rank, world)
        try:
            metadata = transport.metadata() if rank == 0 else None
            meta_box[rank] = metadata
            barrier.wait(10)
            md = meta_box[0]
            # first exchange: rank 0 -> ranks 1, 2
            if rank == 0:
                transport.send_checkpoint([1, 2], step=1, state_dict=want, timeout=timeout)
            else:
                got = transport.recv_checkpoint(0, md, step=1, timeout=timeout)
                assert_state_equal(got, want)
            barrier.wait(10)
            transport.disallow_checkpoint()
            # second exchange: rank 0 -> rank 1
            if rank == 0:
                transport.send_checkpoint([1], step=2, state_dict=want, timeout=timeout)
            elif rank == 1:
                assert_state_equal(transport.recv_checkpoint(0, md, step=2, timeout=timeout), want)
            barrier.wait(10)
            transport.disallow_checkpoint()
            # third exchange: nobody sends; the receiver must give up quickly
            if rank == 2:
                with pytest.raises(Exception):
                    transport.recv_checkpoint(0, md, step=3, timeout=timedelta(milliseconds=10))
            barrier.wait(10)
        finally:
            transport.shutdown(wait=False)
        return True

    meta_box = {}
    with ThreadPoolExecutor(max_workers=world) as ex:
        futs = [ex.submit(run, r) for r in range(world)]
        assert all(f.result(timeout=60) for f in futs)


@pytest.mark.parametrize("chunks", [0, 3])
def test_http_transport_multi_recovery(chunks):
    run_multi_recovery(lambda rank, world: HTTPTransport(timedelta(seconds=10), num_chunks=chunks))


def test_http_transport_wrong_step_and_lock_state():
    t = HTTPTransport(timedelta(seconds=1), num_chunks=0)
    try:
        assert t._lock.w_locked()  # nothing is served before the first send
        t.send_checkpoint([1], step=5, state_dict={"a": torch.ones(2)}, timeout=timedelta(seconds=1))
        assert not t._lock.w_locked()
        url = t.metadata().replace(__import__("socket").gethostname(), "localhost")
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(url + "6/full", timeout=2)
        assert e.value.code == 400
        got = t.recv_checkpoint(0, t.metadata(), 5, timedelta(seconds=2))
        torch.testing.assert_close(got["a"], torch.ones(2))
        t.disallow_checkpoint()
        t.disallow_checkpoint()  # idempotent
        assert t._lock.w_locked()
        t.allow_checkpoint(6)
        assert not t._lock.w_locked()
    finally:
        t.shutdown()


def _gloo_pgs(world):
    store = dist.TCPStore("localhost", 0, is_master=True, wait_for_workers=False)
    addr = f"localhost:{store.port}/prefix"
    pgs = [ProcessGroupGloo(timeout=timedelta(seconds=10)) for _ in range(world)]
    with ThreadPoolExecutor(max_workers=world) as ex:
        list(ex.map(lambda r: pgs[r].configure(addr, "rep", r, world), range(world)))
    return store, pgs


@pytest.mark.parametrize("inplace", [False, True])
def test_pg_transport_gloo(inplace):
    world = 3
    store, pgs = _gloo_pgs(world)
    try:
        def init(rank, world):
            sd = (lambda: make_state(99)) if inplace else None
            return PGTransport(pgs[rank], timedelta(seconds=10), torch.device("cpu"), state_dict=sd)

        run_multi_recovery(init, world)
    finally:
        for pg in pgs:
            pg.shutdown()


def test_transport_benchmark_smoke(capsys):
    """The transport benchmark with a few hundred bytes, as a smoke test of its HTTP path
    (torchft/checkpointing/http_transport_test.py:138-146 does the same with the reference's bench)."""
    import sys as _sys
    from unittest.mock import patch as _patch

    from torchft_b200.checkpointing import bench_transports as B

    for chunks in ("0", "2"):
        with _patch.object(_sys, "argv", ["bench_transports", "--transport", "http", "--total-mb", "0.0004", "--chunk-mb",
                                          "0.0001", "--num-chunks", chunks, "--timeout", "10"]):
            assert B.main() == 0
    assert '"transport": "http"' in capsys.readouterr().out


def test_durable_checkpointer_roundtrip_prune_and_incomplete(tmp_path):
    """Durable checkpoints: atomic per-rank files, a step is usable only when every rank wrote it, old steps are
    pruned, and a fresh process restores model, optimizer and the manager's step from the newest complete one."""
    from unittest.mock import MagicMock

    from torchft_b200.checkpointing.durable import DurableCheckpointer

    def fake_manager(step):
        m = MagicMock()
        state = {"step": step, "batches_committed": 2 * step}
        m.current_step.side_effect = lambda: state["step"]
        m.state_dict.side_effect = lambda: dict(state)
        m.load_state_dict.side_effect = lambda sd: state.update(sd)
        m._user_state_dicts = {}
        m._load_state_dict_fns = {}
        m._state = state
        return m

    w = torch.arange(6, dtype=torch.float32)
    m0 = fake_manager(0)
    m0._user_state_dicts["trainer"] = lambda: {"w": w.clone()}
    ck0 = DurableCheckpointer(m0, str(tmp_path), rank=0, world_size=2, every=2, keep=2)
    ck1 = DurableCheckpointer(m0, str(tmp_path), rank=1, world_size=2, every=2, keep=2)
    assert ck0.maybe_save() is None and ck0.load_latest() is None  # step 0: nothing to do, nothing to load
    for step in (1, 2, 3, 4, 5, 6):
        m0._state.update(step=step, batches_committed=2 * step)
        w.add_(1)
        wrote = ck0.maybe_save(extra={"loader_pos": 10 * step})
        assert (wrote is not None) == (step % 2 == 0)
        if step != 6:
            ck1.maybe_save()  # rank 1 never writes step 6: that step stays incomplete
        assert ck0.maybe_save() is None  # once per step
    assert ck0.complete_steps() == [2, 4]
    ck0.save()  # re-saving by rank 0 prunes by complete steps only
    assert not list(tmp_path.glob("**/*.tmp*"))

    got = {}
    m1 = fake_manager(0)
    m1._load_state_dict_fns["trainer"] = lambda sd: got.update(sd)
    extra = DurableCheckpointer(m1, str(tmp_path), rank=0, world_size=2).load_latest()
    assert extra == {"loader_pos": 40} and m1._state == {"step": 4, "batches_committed": 8}
    torch.testing.assert_close(got["w"], torch.arange(6, dtype=torch.float32) + 4)
    # pruning keeps the newest `keep` complete steps
    m0._state.update(step=8, batches_committed=16)
    ck1.save()
    ck0.save()
    assert ck0.complete_steps() == [4, 8]


def test_durable_checkpoint_resumes_a_real_trainer(tmp_path):
    """Train a few fault-tolerant steps, checkpoint, start over in a fresh manager + trainer, resume: the weights,
    the optimizer state and the manager's step come back and the next step matches an uninterrupted run."""
    from torch.distributed import TCPStore

    from torchft_b200 import Manager, ProcessGroupGloo
    from torchft_b200._ftcp import LighthouseServer
    from torchft_b200.checkpointing.durable import DurableCheckpointer
    from torchft_b200.models.llama import LLAMA_TINY
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer

    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10, heartbeat_timeout_ms=500)
    cfg, B, S = LLAMA_TINY, 1, 16

    def make(replica_id):
        store = TCPStore("localhost", 0, is_master=True, wait_for_workers=False)
        manager = Manager(pg=ProcessGroupGloo(timeout=timedelta(seconds=10)), min_replica_size=1, load_state_dict=None,
                          state_dict=None, replica_id=replica_id, store_addr="localhost", store_port=store.port, rank=0,
                          world_size=1, lighthouse_addr=lh.address(), port=0, timeout=timedelta(seconds=10),
                          quorum_timeout=timedelta(seconds=20), connect_timeout=timedelta(seconds=10), hostname="localhost")
        tr = ShardedLlamaTrainer(cfg, B, S, torch.device("cpu"), manager=manager, seed=3, lr=1e-2)
        manager.register_state_dict_fn("trainer", tr.load_state_dict, tr.state_dict)
        return store, manager, tr

    def batch(step):
        g = torch.Generator().manual_seed(step)
        t = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g)
        return t[:, :-1], t[:, 1:]

    managers = []
    try:
        _, m_a, tr_a = make("durable_a")
        managers.append(m_a)
        ck = DurableCheckpointer(m_a, str(tmp_path), rank=0, world_size=1, every=2)
        for step in range(4):
            tr_a.train_step(*batch(step))
            ck.maybe_save(extra={"next_batch": step + 1})
        assert ck.complete_steps() == [2, 4]
        tr_a.train_step(*batch(4))  # the uninterrupted run goes one step further
        m_a.shutdown(wait=False)  # the whole job goes away (its heartbeats must stop before a new one can form a quorum)
        time.sleep(0.3)

        _, m_b, tr_b = make("durable_b")
        managers.append(m_b)
        extra = DurableCheckpointer(m_b, str(tmp_path), rank=0, world_size=1).load_latest()
        assert extra == {"next_batch": 4} and m_b.current_step() == 4 and tr_b.opt_step == 4
        tr_b.train_step(*batch(extra["next_batch"]))
        assert m_b.current_step() == 5
        for u in range(cfg.n_units):
            torch.testing.assert_close(tr_b.master[u], tr_a.master[u])
            torch.testing.assert_close(tr_b.v[u], tr_a.v[u])
    finally:
        for m in managers:
            m.shutdown(wait=False)
        lh.shutdown()


def test_streaming_serialisation_roundtrip_and_framing():
    """The transports' stream format: nested containers, every dtype incl. bf16, scalars, empty and
    non-contiguous tensors, Python leaves; reads from a stream that returns short reads; rejects garbage."""
    import io

    from torch.utils._pytree import tree_flatten

    from torchft_b200.checkpointing._serialization import streaming_load, streaming_save

    sd = {
        "model": {"w": torch.randn(5, 7), "b": torch.randn(7).bfloat16(), "idx": torch.arange(10)[::2],
                  "half": torch.randn(3, 3).half(), "flag": torch.tensor(True), "empty": torch.empty(0, 4)},
        "optim": [torch.tensor(3.5), {"step": 7, "name": "adamw", "nested": (1, 2.0, None)}],
        "param": torch.nn.Parameter(torch.ones(2, 2)),
    }
    buf = io.BytesIO()
    streaming_save(sd, buf)

    class Dribble(io.RawIOBase):  # a socket that hands out at most 1000 bytes at a time
        def __init__(self, data):
            self.data, self.pos = data, 0

        def readable(self):
            return True

        def readinto(self, b):
            n = min(len(b), 1000, len(self.data) - self.pos)
            b[:n] = self.data[self.pos : self.pos + n]
            self.pos += n
            return n

    for stream in (io.BytesIO(buf.getvalue()), io.BufferedReader(Dribble(buf.getvalue()), 4096), Dribble(buf.getvalue())):
        got = streaming_load(stream)
        a, spec_a = tree_flatten(sd)
        b, spec_b = tree_flatten(got)
        assert spec_a == spec_b
        for x, y in zip(a, b):
            if isinstance(x, torch.Tensor):
                assert x.dtype == y.dtype and x.shape == y.shape and torch.equal(x.detach(), y)
            else:
                assert x == y
    with pytest.raises(ValueError):
        streaming_load(io.BytesIO(b"garbage-garbage-garbage"))
    with pytest.raises(EOFError):
        streaming_load(io.BytesIO(buf.getvalue()[:-5]))


@pytest.mark.parametrize("num_chunks", [0, 3])
def test_http_transport_receives_in_place(num_chunks):
    """With a `state_dict` callable the HTTP transport fills matching tensors in place (and falls back to new
    tensors where shape or dtype differ)."""
    timeout = timedelta(seconds=10)
    src = {"a": torch.arange(12, dtype=torch.float32).reshape(3, 4), "b": torch.ones(5).bfloat16(), "n": 7,
           "c": torch.full((2, 2), 3.0), "d": torch.arange(4)}
    dst = {"a": torch.zeros(3, 4), "b": torch.zeros(5).bfloat16(), "n": 0, "c": torch.zeros(3, 3), "d": torch.zeros(4)}
    send = HTTPTransport(timeout, num_chunks=num_chunks)
    recv = HTTPTransport(timeout, num_chunks=num_chunks, state_dict=lambda: dst)
    try:
        send.send_checkpoint([1], step=3, state_dict=src, timeout=timeout)
        got = recv.recv_checkpoint(0, send.metadata(), 3, timeout)
        assert got["a"] is dst["a"] and got["b"] is dst["b"]  # filled in place
        assert got["c"] is not dst["c"] and got["d"] is not dst["d"]  # shape / dtype mismatch: fresh tensors
        for k in ("a", "b", "c", "d"):
            assert torch.equal(got[k], src[k])
        assert got["n"] == 7
    finally:
        send.shutdown()
        recv.shutdown()


def test_transports_carry_dtensor_leaves():
    """A state dict with DTensor leaves (what FSDP2 / tensor-parallel models hold) survives the HTTP and the
    process-group transport: the local shard travels, the receiver gets a DTensor on its own mesh again
    (the reference's transport tests include a DTensor leaf, torchft/checkpointing/transport_test.py:45-155).
    Runs in a child because it initialises torch.distributed."""
    import subprocess
    import sys

    child = r'''
import threading, torch, torch.distributed as dist
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.tensor import DTensor, Shard, distribute_tensor
from torchft_b200.checkpointing.http_transport import HTTPTransport
from torchft_b200.checkpointing.pg_transport import PGTransport
from torchft_b200.process_group import ProcessGroupGloo

store = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
dist.init_process_group("gloo", store=dist.PrefixStore("w", store), rank=0, world_size=1)
mesh = init_device_mesh("cpu", (1,))
full = torch.arange(12, dtype=torch.float32).reshape(4, 3)
sd = {"dt": distribute_tensor(full, mesh, [Shard(0)]), "plain": torch.ones(2), "s": "x", "i": 3}
timeout = timedelta(seconds=10)

def check(got):
    assert isinstance(got["dt"], DTensor), type(got["dt"])
    assert got["dt"].placements == sd["dt"].placements and tuple(got["dt"].shape) == (4, 3)
    torch.testing.assert_close(got["dt"].to_local(), full)
    torch.testing.assert_close(got["plain"], torch.ones(2))
    assert got["s"] == "x" and got["i"] == 3

send, recv = HTTPTransport(timeout, num_chunks=0), HTTPTransport(timeout, num_chunks=0)
send.send_checkpoint([1], 1, sd, timeout)
check(recv.recv_checkpoint(0, send.metadata(), 1, timeout))
send.shutdown(); recv.shutdown()

pgs = [ProcessGroupGloo(timeout=timeout) for _ in range(2)]
with ThreadPoolExecutor(2) as ex:
    list(ex.map(lambda r: pgs[r].configure(f"127.0.0.1:{store.port}/t", "rep", r, 2), range(2)))
trs = [PGTransport(pgs[r], timeout, torch.device("cpu")) for r in range(2)]
with ThreadPoolExecutor(2) as ex:
    f0 = ex.submit(trs[0].send_checkpoint, [1], 1, sd, timeout)
    f1 = ex.submit(trs[1].recv_checkpoint, 0, trs[0].metadata(), 1, timeout)
    f0.result(30); check(f1.result(30))
# in place: the receiver's own DTensor gets the values
mine = {"dt": distribute_tensor(torch.zeros(4, 3), mesh, [Shard(0)]), "plain": torch.zeros(2), "s": "", "i": 0}
trs[1] = PGTransport(pgs[1], timeout, torch.device("cpu"), state_dict=lambda: mine)
with ThreadPoolExecutor(2) as ex:
    f0 = ex.submit(trs[0].send_checkpoint, [1], 2, sd, timeout)
    f1 = ex.submit(trs[1].recv_checkpoint, 0, trs[0].metadata(), 2, timeout)
    f0.result(30); check(f1.result(30))
torch.testing.assert_close(mine["dt"].to_local(), full)
for pg in pgs: pg.shutdown()
print("dtensor ok")
'''
    import os as _os
    repo = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", child], capture_output=True, text=True, timeout=240,
                       env=dict(_os.environ, PYTHONPATH=repo))
    assert r.returncode == 0 and "dtensor ok" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
