"""OptimizerWrapper, DistributedSampler, DDP wrappers, ParameterServer, coordination
docstrings, structured loggers, launcher plumbing."""
import json
import logging
import threading
from datetime import timedelta
from unittest.mock import MagicMock, create_autospec

import pytest
import torch
from torch import nn, optim
from torch.distributed.distributed_c10d import ReduceOp

from torchft_b200 import coordination
from torchft_b200.data import DistributedSampler
from torchft_b200.ddp import DistributedDataParallel, PureDistributedDataParallel
from torchft_b200.manager import Manager
from torchft_b200.optim import OptimizerWrapper
from torchft_b200.parameter_server import ParameterServer
from torchft_b200.process_group import ProcessGroup, ProcessGroupGloo
from torchft_b200.work import _DummyWork


def test_optimizer_wrapper_gates_step():
    manager = create_autospec(Manager, instance=True)
    model = nn.Linear(3, 4)
    inner = optim.SGD(model.parameters(), lr=1.0)
    opt = OptimizerWrapper(manager, inner)
    opt.zero_grad()
    assert manager.start_quorum.call_count == 1
    before = model.weight.detach().clone()
    model(torch.ones(2, 3)).sum().backward()
    manager.should_commit.return_value = False
    opt.step()
    assert torch.equal(model.weight, before)
    manager.should_commit.return_value = True
    opt.step()
    assert not torch.equal(model.weight, before)
    assert opt.param_groups is inner.param_groups and opt.state is inner.state
    opt.load_state_dict(opt.state_dict())
    opt.add_param_group({"params": [nn.Parameter(torch.zeros(1))]})
    assert len(inner.param_groups) == 2
    with pytest.raises(AssertionError):
        opt.step(closure=lambda: 0)


def test_distributed_sampler_sharding():
    data = list(range(1000))
    s = DistributedSampler(data, replica_rank=1, num_replica_groups=2, group_rank=3, num_replicas=4, shuffle=False)
    assert s.global_rank == 3 + 4 * 1 and s.global_world_size == 8
    idx = list(iter(s))
    assert idx[0] == 7 and idx[1] == 15 and len(idx) == 125


def _mock_manager():
    m = create_autospec(Manager, instance=True)
    m.allreduce.side_effect = lambda t, should_quantize=False, reduce_op=ReduceOp.AVG: _DummyWork(t)
    return m


def test_ddp_calls_manager_allreduce_per_bucket():
    m = _mock_manager()
    model = nn.Sequential(nn.Linear(3, 4), nn.Linear(4, 2))
    ddp = DistributedDataParallel(m, model)
    ddp(torch.ones(5, 3)).sum().backward()
    assert m.allreduce.call_count >= 1
    assert all(p.grad is not None for p in model.parameters())


def test_pure_ddp_one_allreduce_per_parameter():
    m = _mock_manager()
    model = nn.Sequential(nn.Linear(3, 4), nn.Linear(4, 2))
    ddp = PureDistributedDataParallel(m, model)
    ddp(torch.ones(5, 3)).sum().backward()
    assert m.allreduce.call_count == len(list(model.parameters()))


def test_parameter_server_session():
    class PS(ParameterServer):
        @classmethod
        def new_process_group(cls) -> ProcessGroup:
            return ProcessGroupGloo(timeout=timedelta(seconds=10))

        def forward(self, session_id: str, pg: ProcessGroup) -> None:
            t = torch.zeros(3)
            pg.broadcast_one(t, root=1).wait()       # client -> server
            pg.broadcast_one(t * 2, root=0).wait()   # server -> client
            pg.shutdown()

    ps = PS(port=0)
    try:
        pg = PS.new_session(ps.address())
        x = torch.arange(3.0)
        pg.broadcast_one(x, root=1).wait()
        out = torch.zeros(3)
        pg.broadcast_one(out, root=0).wait()
        assert torch.equal(out, x * 2)
        pg.shutdown()
    finally:
        ps.shutdown()


def test_coordination_api_is_documented():
    # every exported class and function explains its arguments (the check of torchft/coordination_test.py)
    for name in coordination.__all__:
        doc = getattr(coordination, name).__doc__ or ""
        assert "Args" in doc, name
    assert "Args:" in coordination.__doc__


def test_structured_loggers_carry_fields():
    from torchft_b200.otel import _FieldFormatter, setup_logger

    lg = setup_logger("torchft_commits")
    records = []

    class H(logging.Handler):
        def emit(self, r):
            records.append(r)

    h = H()
    lg.addHandler(h)
    try:
        lg.info("", extra={"job_id": "j", "replica_id": "r", "rank": 0, "quorum_id": 3, "step": 9, "commit_result": True})
    finally:
        lg.removeHandler(h)
    line = _FieldFormatter().format(records[0])
    assert "quorum_id=3" in line and "commit_result=True" in line and "step=9" in line


def test_runner_environment_and_punisher(tmp_path):
    from torchft_b200.launch.runner import Punisher, Runner

    r = Runner(["train.py"], num_groups=2, gpus_per_group=4, lighthouse_addr="http://x:1", pid_file=str(tmp_path / "p.json"))
    env = r._env(1)
    assert env["REPLICA_GROUP_ID"] == "1" and env["NUM_REPLICA_GROUPS"] == "2" and env["CUDA_VISIBLE_DEVICES"] == "4,5,6,7"
    (tmp_path / "p.json").write_text(json.dumps({"0": None, "1": None}))
    assert Punisher(str(tmp_path / "p.json")).kill_one() is None


# ---- pieces added with the engine-native DiLoCo and the attention kernels -------------------


def test_split_units_is_contiguous_balanced_and_total():
    from torchft_b200.parallel.diloco import split_units

    numels = [500, 10, 10, 10, 10, 10, 10, 10, 10, 520]
    parts = split_units(numels, 4)
    assert [u for p in parts for u in p] == list(range(len(numels)))  # contiguous cover
    assert all(parts)
    assert parts[0] == [0] and parts[-1][-1] == 9
    assert split_units([1, 1, 1], 3) == [[0], [1], [2]]
    import pytest as _pytest

    with _pytest.raises(ValueError):
        split_units([1, 2], 3)


def test_engine_diloco_argument_validation():
    from unittest.mock import MagicMock

    import pytest as _pytest
    import torch as _torch

    from torchft_b200.models.llama import LLAMA_TINY
    from torchft_b200.parallel.diloco import EngineDiLoCo
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer

    tr = ShardedLlamaTrainer(LLAMA_TINY, 1, 16, _torch.device("cpu"))
    m = MagicMock()
    m._use_async_quorum = True
    with _pytest.raises(ValueError):
        EngineDiLoCo(tr, m, n_fragments=2, sync_every=4)  # needs a synchronous quorum
    m._use_async_quorum = False
    with _pytest.raises(ValueError):
        EngineDiLoCo(tr, m, n_fragments=3, sync_every=4)  # not a multiple
    with _pytest.raises(ValueError):
        EngineDiLoCo(tr, m, n_fragments=2, sync_every=4, fragment_sync_delay=2)  # delay >= interval
    with _pytest.raises(ValueError):
        EngineDiLoCo(tr, m, n_fragments=2, sync_every=4, fragment_update_alpha=1.5)
    d = EngineDiLoCo(tr, m, n_fragments=2, sync_every=4)
    assert len(d.fragments) == 2 and m.register_state_dict_fn.call_count == 2
    tr2 = ShardedLlamaTrainer(LLAMA_TINY, 1, 16, _torch.device("cpu"), manager=m)
    with _pytest.raises(ValueError):
        EngineDiLoCo(tr2, m, n_fragments=2, sync_every=4)  # the trainer must not allreduce every step


def test_attention_selection_and_cpu_wrappers():
    import pytest as _pytest
    import torch as _torch

    from torchft_b200.models.llama import LLAMA3_8B, LLAMA_TINY, SdpaAttention, make_attention
    from torchft_b200.ops import kernels as K

    cpu = _torch.device("cpu")
    assert isinstance(make_attention(LLAMA3_8B, 8192, cpu), SdpaAttention)  # no CUDA: library/CPU path
    assert isinstance(make_attention(LLAMA_TINY, 128, cpu, "sdpa"), SdpaAttention)
    with _pytest.raises(ValueError):
        make_attention(LLAMA_TINY, 128, cpu, "tcgen05")
    assert K.attention_supported(8192, 128) and K.attention_supported(2048, 64) and not K.attention_supported(100, 128)
    assert not K.attention_supported(128, 64) and not K.attention_supported(8192, 96)
    # the CPU restatement behind the wrappers: forward + backward agree with autograd of the reference
    B, S, Hq, Hkv, D = 1, 8, 2, 1, 4
    g = _torch.Generator().manual_seed(0)
    qkv = _torch.randn(B * S, (Hq + 2 * Hkv) * D, generator=g).bfloat16()
    q, k, v = qkv[:, : Hq * D], qkv[:, Hq * D : (Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D :]
    out = _torch.empty(B * S, Hq * D, dtype=_torch.bfloat16)
    lse = _torch.empty(B, Hq, S)
    K.attention_fwd(q, k, v, B, S, Hq, Hkv, D, out, lse)
    assert _torch.isfinite(out.float()).all() and _torch.isfinite(lse).all()
    dqkv = _torch.zeros_like(qkv)
    K.attention_bwd(q, k, v, out, _torch.ones_like(out), lse, dqkv[:, : Hq * D], dqkv[:, Hq * D : (Hq + Hkv) * D],
                    dqkv[:, (Hq + Hkv) * D :], B, S, Hq, Hkv, D)
    assert dqkv.float().abs().sum() > 0


def test_open_group_store():
    """Every rank of a replica group learns the ephemeral port of its group's store; groups get
    different stores (4 gloo ranks = 2 groups of 2)."""
    import json
    import os
    import socket
    import subprocess
    import sys

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_group_store_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "4", "2", str(port)], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(4)]
    res = []
    for p in procs:
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0, err[-2000:]
        res.append(json.loads([l for l in out.splitlines() if l.startswith("{")][-1]))
    res.sort(key=lambda r: r["rank"])
    assert res[0]["port"] == res[1]["port"] and res[2]["port"] == res[3]["port"] and res[0]["port"] != res[2]["port"]
    assert [r["who"] for r in res] == ["group0", "group0", "group1", "group1"]


def test_bench_reference_arm():
    """`bench.py --impl reference` runs the unmodified reference package (a copy under baseline/_ref) on the pure-Python
    control-plane stand-in.  Without a GPU it prints one `unavailable` line and exits 0; with `FTB200_REF_DEVICE=cpu` the
    same path runs a tiny model over Gloo, which checks the stand-in and the reference's manager, optimizer wrapper and
    managed process group end to end."""
    import json
    import os
    import subprocess
    import sys

    import pytest

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.isdir(os.path.join(root, "baseline", "_ref", "torchft")):
        pytest.skip("no copy of the reference package under baseline/_ref")
    cmd = [sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"]
    import torch

    if not torch.cuda.is_available():
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-1000:]
        line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
        assert line["impl"] == "reference" and "no CUDA device" in line["unavailable"]
    env = dict(os.environ, FTB200_REF_DEVICE="cpu")
    r = subprocess.run(cmd + ["--model", "debug", "--seq-len", "64"], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-1500:]
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["commits"] == 4 and line["value"] > 0, line
    assert "stand-in" in line["control_plane"]


def test_thread_backed_mp_context_pipe_and_process():
    """DummyContext: pipes with timeouts and EOF, a 'process' that is a thread, fd-like sharing of an endpoint."""
    import threading
    from datetime import timedelta

    from torchft_b200.multiprocessing import _MonitoredPipe
    from torchft_b200.multiprocessing_dummy_context import DummyContext, get_context

    ctx = get_context("spawn")
    assert isinstance(ctx, DummyContext) and ctx.get_start_method() == "thread"
    parent, child = ctx.Pipe()

    def echo(conn, tag):
        try:
            while True:
                conn.send((tag, conn.recv()))
        except (EOFError, OSError):
            pass

    p = ctx.Process(target=echo, args=(child, "x"), daemon=True)
    p.start()
    child.close()  # the parent's copy, as after a fork: the worker's stays open
    mon = _MonitoredPipe(parent)
    mon.send(41)
    assert mon.recv(timedelta(seconds=5)) == ("x", 41)
    with pytest.raises(TimeoutError):
        mon.recv(timedelta(milliseconds=50))
    assert p.is_alive() and p.pid is not None
    payload = object()
    mon.send(payload)
    assert mon.recv(timedelta(seconds=5))[1] is payload  # by reference, nothing is pickled
    mon.close()  # EOF for the worker
    p.join(5)
    assert not p.is_alive() and p.exitcode == 0

    # kill() unblocks a worker that waits on its endpoint
    a, b = ctx.Pipe()
    q = ctx.Process(target=echo, args=(b, "y"))
    q.start()
    q.kill()
    q.join(5)
    assert not q.is_alive()
    with pytest.raises((EOFError, OSError)):
        a.recv()
    assert isinstance(ctx.Lock(), type(threading.Lock())) and ctx.Queue().empty() and not ctx.Event().is_set()


def test_optimizer_wrapper_reports_commit_and_works_with_lr_schedulers():
    manager = create_autospec(Manager, instance=True)
    model = nn.Linear(2, 2)
    inner = optim.SGD(model.parameters(), lr=1.0)
    opt = OptimizerWrapper(manager, inner)
    assert opt.last_step_committed is None and "SGD" in repr(opt)
    sched = torch.optim.lr_scheduler.StepLR(opt, step_size=1, gamma=0.5)  # schedulers accept the wrapper
    for commit in (True, False, True):
        manager.should_commit.return_value = commit
        opt.zero_grad()
        model(torch.ones(1, 2)).sum().backward()
        opt.step()
        assert opt.last_step_committed is commit
        sched.step()
    assert inner.param_groups[0]["lr"] == 0.125 and opt.defaults is inner.defaults
    seen = []
    handle = opt.register_step_post_hook(lambda o, a, k: seen.append(type(o).__name__))  # hooks live on the real optimizer
    manager.should_commit.return_value = True
    opt.step()
    handle.remove()
    assert seen == ["SGD"]


def test_extension_stub_matches_the_module():
    """torchft_b200/_ftcp.pyi names exactly the classes, methods, attributes and functions the extension module has,
    with the same parameter names."""
    import ast
    import inspect
    import re
    from pathlib import Path

    from torchft_b200 import _ftcp as C

    tree = ast.parse((Path(C.__file__).parent / "_ftcp.pyi").read_text())
    stub_classes = {n.name: n for n in tree.body if isinstance(n, ast.ClassDef)}
    stub_funcs = {n.name: n for n in tree.body if isinstance(n, ast.FunctionDef)}
    real_classes = {n: o for n, o in vars(C).items() if inspect.isclass(o)}
    real_funcs = {n: o for n, o in vars(C).items() if callable(o) and not inspect.isclass(o) and not n.startswith("__")}
    assert set(stub_classes) == set(real_classes)
    assert set(stub_funcs) == set(real_funcs)

    def params(doc):  # "name(self: X, a: int, b: str = '') -> R" -> ["a", "b"]
        inside = doc.strip().splitlines()[0]
        inside = inside[inside.index("(") + 1:inside.rindex(")")]
        names = re.findall(r"(?:^|, )(\w+): ", inside)
        return [n for n in names if n != "self"]

    for name, node in stub_classes.items():
        real = real_classes[name]
        stub_members = {m.name for m in node.body if isinstance(m, ast.FunctionDef)} | {
            m.target.id for m in node.body if isinstance(m, ast.AnnAssign)}
        real_members = {m for m in vars(real) if not m.startswith("__") and "pybind11" not in m} | {"__init__"}
        assert stub_members == real_members, (name, stub_members ^ real_members)
        for m in node.body:
            if isinstance(m, ast.FunctionDef):
                want = params(getattr(real, m.name).__doc__)
                got = [a.arg for a in m.args.args if a.arg != "self"]
                assert got == want, (name, m.name, got, want)
    for name, node in stub_funcs.items():
        want = params(real_funcs[name].__doc__)
        got = [a.arg for a in node.args.args]
        assert got == want or name == "quorum_changed", (name, got, want)
