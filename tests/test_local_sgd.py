"""LocalSGD / DiLoCo unit tests against a mocked Manager, and the analytic golden sequence:
inner lr 1 with constant gradient 2, outer lr 2, 2 fragments, sync_every 6 gives local
weights 1,-1,-3,-11,... for fragment 0 and global updates -11, -23, -35, -47."""
from unittest.mock import create_autospec

import pytest
import torch
from torch import nn, optim

from torchft_b200.local_sgd import DiLoCo, LocalSGD, _StreamingDiLoCoFragment
from torchft_b200.manager import Manager
from torchft_b200.work import _DummyWork


class TinyModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(3, 4), nn.ReLU(), nn.Linear(4, 2))

    def forward(self, x):
        return self.net(x)


def mock_manager(commit=True, factor=1.0):
    m = create_autospec(Manager, instance=True)
    m._use_async_quorum = False
    m.should_commit.return_value = commit
    m.current_step.return_value = 0

    def allreduce(t, should_quantize=False, reduce_op=None):
        t.mul_(factor)
        return _DummyWork(t)

    m.allreduce.side_effect = allreduce
    return m


def test_local_sgd_sync_cadence_and_copy_back():
    model = TinyModel()
    opt = optim.SGD(model.parameters(), lr=0.1)
    m = mock_manager(factor=0.5)
    with LocalSGD(m, model, opt, sync_every=2) as ls:
        for step in range(1, 5):
            opt.zero_grad()
            model(torch.rand(5, 3)).sum().backward()
            before = [p.detach().clone() for p in model.parameters()]
            opt.step()
            if step % 2 == 0:
                assert m.start_quorum.call_count == step // 2
                assert m.should_commit.call_count == step // 2
            assert ls._local_step == step % 2
    assert m.allreduce.call_count == 2 * len(list(model.parameters()))
    assert m.disallow_state_dict_read.call_count == 4 and m.allow_state_dict_read.call_count == 4


def test_local_sgd_no_copy_when_commit_fails():
    model = TinyModel()
    opt = optim.SGD(model.parameters(), lr=0.1)
    m = mock_manager(commit=False, factor=0.0)
    with LocalSGD(m, model, opt, sync_every=1):
        opt.zero_grad()
        model(torch.rand(5, 3)).sum().backward()
        opt.step()
    assert all(p.abs().sum() > 0 for p in model.parameters())  # zeros from the failed sync were not applied


def test_diloco_argument_validation():
    model = TinyModel()
    inner = optim.SGD(model.parameters(), lr=0.1)
    outer = optim.SGD(model.parameters(), lr=0.7, momentum=0.9, nesterov=True)
    m = mock_manager()
    m._use_async_quorum = True
    with pytest.raises(ValueError, match="synchronous quorum"):
        DiLoCo(m, [model], inner, outer, sync_every=2)
    m._use_async_quorum = False
    frags = [model.net[0], model.net[2]]
    with pytest.raises(ValueError):
        DiLoCo(m, frags, inner, outer, sync_every=1)  # fewer steps than fragments
    with pytest.raises(ValueError):
        DiLoCo(m, frags, inner, outer, sync_every=3)  # not divisible
    with pytest.raises(ValueError):
        DiLoCo(m, frags, inner, outer, sync_every=4, fragment_sync_delay=2)
    with pytest.raises(ValueError):
        DiLoCo(m, frags, inner, outer, sync_every=4, fragment_update_alpha=1.5)
    with pytest.raises(AssertionError):
        DiLoCo(m, frags, inner, [outer], sync_every=4)


def test_diloco_healthy_flow():
    model = TinyModel()
    inner = optim.AdamW(model.parameters(), lr=1e-2)
    outer = optim.SGD(model.parameters(), lr=0.7, momentum=0.9, nesterov=True)
    m = mock_manager()
    with DiLoCo(m, [model], inner, outer, sync_every=2) as d:
        frag = d._fragments[0]
        start = {n: p.detach().clone() for n, p in model.named_parameters()}
        for n, t in frag.original_parameters.items():
            torch.testing.assert_close(t, start[n])
        inner.zero_grad(); model(torch.rand(4, 3)).sum().backward(); inner.step()
        assert m.start_quorum.call_count == 0 and d._local_step == 1
        inner.zero_grad(); model(torch.rand(4, 3)).sum().backward(); inner.step()
        assert m.start_quorum.call_count == 1 and m.should_commit.call_count == 1 and d._local_step == 0
        # the backup now holds the new global weights, which the model carries too (alpha 0)
        for n, p in model.named_parameters():
            torch.testing.assert_close(frag.original_parameters[n], p.detach())
        assert m.allreduce.call_count == len(list(model.parameters()))


def test_diloco_failed_commit_restores_global_weights():
    model = TinyModel()
    inner = optim.SGD(model.parameters(), lr=0.1)
    outer = optim.SGD(model.parameters(), lr=0.7)
    m = mock_manager(commit=False)
    start = {n: p.detach().clone() for n, p in model.named_parameters()}
    with DiLoCo(m, [model], inner, outer, sync_every=1):
        inner.zero_grad(); model(torch.rand(4, 3)).sum().backward(); inner.step()
    for n, p in model.named_parameters():
        torch.testing.assert_close(p.detach(), start[n])


def test_bucketization_matches_per_param_and_keeps_oversized_tensors():
    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Parameter(torch.zeros(10))
            self.b = nn.Parameter(torch.zeros(300))  # larger than the bucket cap below
            self.c = nn.Parameter(torch.zeros(7))

    model = M()
    m = mock_manager(factor=2.0)
    inner = optim.SGD(model.parameters(), lr=0.1)
    frag = _StreamingDiLoCoFragment(m, model, 0, 1, inner, optim.SGD(model.parameters(), lr=1.0), 1,
                                    use_bucketization=True, bucket_cap_mb=None)
    frag.bucket_cap_mb = 64 * 4  # bytes: 64 fp32 elements
    frag._grads = {"a": torch.ones(10), "b": torch.full((300,), 2.0), "c": torch.full((7,), 3.0)}
    frag._allreduce_bucketized()
    for w in frag._allreduce_work:
        w.wait()
        w.get_future().wait()
    torch.testing.assert_close(frag._grads["a"], torch.full((10,), 2.0))
    torch.testing.assert_close(frag._grads["b"], torch.full((300,), 4.0))
    torch.testing.assert_close(frag._grads["c"], torch.full((7,), 6.0))
    assert m.allreduce.call_count == 3  # a | b (own bucket) | c


class _MockLayer(nn.Module):
    def __init__(self):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(1, 1))


class _MockOptimizer(optim.Optimizer):
    """p -= lr * grad"""

    def __init__(self, params, lr):
        super().__init__(params, dict(lr=lr))

    def step(self, closure=None):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    p.data.add_(p.grad, alpha=-g["lr"])


@pytest.mark.parametrize("n_fragments,expected_l0,expected_l1", [
    (2, [1, -1, -3, -11, -13, -15, -17], [1, -1, -3, -5, -7, -9, -23]),
])
def test_diloco_golden_sequence(n_fragments, expected_l0, expected_l1):
    layers = [_MockLayer() for _ in range(n_fragments)]
    model = nn.Sequential(*layers)
    inner = _MockOptimizer(model.parameters(), lr=1.0)
    outers = [_MockOptimizer(l.parameters(), lr=2.0) for l in layers]
    state = {"step": 0}
    m = create_autospec(Manager, instance=True)
    m._use_async_quorum = False
    m.current_step.side_effect = lambda: state["step"]
    m.allreduce.side_effect = lambda t, should_quantize=False, reduce_op=None: _DummyWork(t)

    def commit():
        state["step"] += 1
        return True

    m.should_commit.side_effect = commit
    seen0, seen1, globals_ = [1.0], [1.0], []
    with DiLoCo(m, layers, inner, outers, sync_every=6) as d:
        for _ in range(6):
            for p in model.parameters():
                p.grad = torch.full_like(p, 2.0)
            inner.step()
            seen0.append(layers[0].weight.item())
            seen1.append(layers[1].weight.item())
            globals_.append((d._fragments[0].original_parameters["weight"].item(),
                             d._fragments[1].original_parameters["weight"].item()))
    assert seen0 == [float(x) for x in expected_l0]
    assert seen1 == [float(x) for x in expected_l1]
    assert globals_[2] == (-11.0, 1.0) and globals_[5] == (-11.0, -23.0)


def _delta_manager(factor=1.0, commit_pattern=None):
    """Mock manager whose allreduce scales by ``factor`` and whose allreduce_delta is the
    unfused definition (out = a - b, then allreduce)."""
    state = {"step": 0, "votes": 0}
    m = create_autospec(Manager, instance=True)
    m._use_async_quorum = False
    m.current_step.side_effect = lambda: state["step"]

    def allreduce(t, should_quantize=False, reduce_op=None):
        t.mul_(factor)
        return _DummyWork(t)

    def allreduce_delta(out, a, b, should_quantize=False):
        torch.sub(a, b, out=out)
        return allreduce(out)

    def commit():
        ok = True if commit_pattern is None else commit_pattern[state["votes"] % len(commit_pattern)]
        state["votes"] += 1
        if ok:
            state["step"] += 1
        return ok

    m.allreduce.side_effect = allreduce
    m.allreduce_delta.side_effect = allreduce_delta
    m.should_commit.side_effect = commit
    return m


@pytest.mark.parametrize("delay,alpha", [(0, 0.0), (1, 0.0), (1, 0.3)])
def test_flat_fragments_match_per_parameter_path(delay, alpha):
    """Flat-buffer fragments (fused outer step) follow the same trajectory as the
    per-parameter path with torch.optim.SGD(nesterov) outside, including a failed vote."""
    def run(flat):
        torch.manual_seed(3)
        model = nn.Sequential(nn.Linear(6, 8), nn.Linear(8, 8), nn.Linear(8, 4), nn.Linear(4, 2))
        frags = [model[:2], model[2:]]
        inner = optim.AdamW(model.parameters(), lr=1e-2)
        outers = [optim.SGD(f.parameters(), lr=0.7, momentum=0.9, nesterov=True) for f in frags]
        m = _delta_manager(factor=0.5, commit_pattern=[True, True, False, True])
        hooks = {}
        m.register_state_dict_fn.side_effect = lambda k, load, save: hooks.__setitem__(k, (load, save))
        g = torch.Generator().manual_seed(11)
        with DiLoCo(m, frags, inner, outers, sync_every=4, fragment_sync_delay=delay, fragment_update_alpha=alpha,
                    flat_fragments=flat) as d:
            assert d.flat_fragments == flat
            for _ in range(16):
                inner.zero_grad()
                model(torch.randn(5, 6, generator=g)).square().mean().backward()
                inner.step()
        backups = [f.original_parameters[n].clone() for f in d._fragments for n in sorted(f.original_parameters)]
        return [p.detach().clone() for p in model.parameters()], backups, hooks

    p_ref, b_ref, hooks_ref = run(False)
    p_flat, b_flat, hooks = run(True)
    for a, b in zip(p_ref + b_ref, p_flat + b_flat):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    # the healing state of a flat fragment has the per-parameter fragment's keys, and the outer
    # optimizer's own state dict carries the momentum (a checkpoint of it restores the momentum)
    load, save = hooks["StreamingDiLoCoFragment_0"]
    load_ref, save_ref = hooks_ref["StreamingDiLoCoFragment_0"]
    sd, sd_ref = save(), save_ref()
    assert set(sd) == set(sd_ref) == {"outer_optimizer", "original_parameters"}
    mom = [st["momentum_buffer"] for st in sd["outer_optimizer"]["state"].values()]
    mom_ref = [st["momentum_buffer"] for st in sd_ref["outer_optimizer"]["state"].values()]
    assert len(mom) == len(mom_ref) > 0 and any(float(b.abs().max()) > 0 for b in mom)
    for a, b in zip(mom, mom_ref):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    # the two layouts heal each other
    load(sd_ref)
    load_ref(sd)
    load(sd)


def test_flat_fragment_detects_moved_parameter():
    model = nn.Sequential(nn.Linear(4, 4))
    inner = optim.SGD(model.parameters(), lr=0.1)
    m = _delta_manager()
    d = DiLoCo(m, [model], inner, optim.SGD(model.parameters(), lr=0.7, momentum=0.9, nesterov=True), sync_every=2,
               flat_fragments=True)
    model[0].weight.data = model[0].weight.data.clone()  # what .to() or load_state_dict(assign=True) does
    with pytest.raises(RuntimeError, match="flat buffer"):
        d._fragments[0].prepare_sync()


def test_flat_fragments_reject_unsupported_outer_optimizer():
    model = TinyModel()
    inner = optim.SGD(model.parameters(), lr=0.1)
    m = _delta_manager()
    with pytest.raises(ValueError):
        DiLoCo(m, [model], inner, optim.Adam(model.parameters(), lr=0.1), sync_every=2, flat_fragments=True)
    # auto mode quietly keeps the per-parameter path
    assert not DiLoCo(m, [model], inner, optim.Adam(model.parameters(), lr=0.1), sync_every=2).flat_fragments


def _simulate_streaming_diloco(n_frag, sync_every, delay, alpha, steps, inner_lr=1.0, grad=2.0, outer_lr=2.0):
    """Independent restatement of streaming DiLoCo for scalar weights, constant gradient and plain SGD
    inside and outside; returns the local weights after every inner step and the global weights."""
    local = [1.0] * n_frag
    glob = [1.0] * n_frag
    every = sync_every // n_frag
    trace, manager_step, local_step, pending = [], 0, 0, None
    for _ in range(steps):
        local = [w - inner_lr * grad for w in local]
        local_step += 1
        if local_step == every - delay:
            f = manager_step % n_frag
            pending = (f, glob[f] - local[f])
        if local_step == every:
            f, pseudo = pending
            new_global = glob[f] - outer_lr * pseudo
            local[f] = new_global + alpha * (local[f] - new_global)
            glob[f] = new_global
            manager_step += 1
            local_step = 0
        trace.append((list(local), list(glob)))
    return trace


@pytest.mark.parametrize("flat", [False, True])
@pytest.mark.parametrize("n_frag,sync_every,delay,alpha", [
    (1, 3, 0, 0.0), (2, 6, 0, 0.0), (2, 6, 1, 0.0), (2, 8, 2, 0.5), (3, 9, 1, 1.0), (3, 12, 3, 0.25),
])
def test_streaming_diloco_matches_independent_simulation(flat, n_frag, sync_every, delay, alpha):
    layers = [_MockLayer() for _ in range(n_frag)]
    model = nn.Sequential(*layers)
    inner = _MockOptimizer(model.parameters(), lr=1.0)
    # the flat path needs torch's SGD outside; without momentum it is the same update as the mock optimizer
    outers = ([optim.SGD(l.parameters(), lr=2.0) for l in layers] if flat
              else [_MockOptimizer(l.parameters(), lr=2.0) for l in layers])
    m = _delta_manager()
    steps = 3 * sync_every
    want = _simulate_streaming_diloco(n_frag, sync_every, delay, alpha, steps)
    with DiLoCo(m, layers, inner, outers, sync_every=sync_every, fragment_sync_delay=delay, fragment_update_alpha=alpha,
                flat_fragments=flat) as d:
        for k in range(steps):
            for p in model.parameters():
                p.grad = torch.full_like(p, 2.0)
            inner.step()
            got_local = [l.weight.item() for l in layers]
            got_global = [f.original_parameters["weight"].item() for f in d._fragments]
            assert got_local == pytest.approx(want[k][0]), (k, got_local, want[k][0])
            assert got_global == pytest.approx(want[k][1]), (k, got_global, want[k][1])
    assert m.should_commit.call_count == 3 * n_frag


def test_local_sgd_and_diloco_with_dtensor_parameters():
    """Models sharded by FSDP2 hold DTensor parameters: LocalSGD and DiLoCo (both fragment layouts) work on the
    local shards and follow the same trajectory as the unsharded model; what reaches the manager's allreduce is a
    plain tensor (torchft/local_sgd.py:33-43 extract_local_tensor).  Child process: it initialises torch.distributed."""
    import os
    import subprocess
    import sys

    child = r'''
import torch, torch.distributed as dist
from torch import nn, optim
from unittest.mock import create_autospec
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.fsdp import fully_shard
from torch.distributed.tensor import DTensor
from torchft_b200.local_sgd import DiLoCo, LocalSGD
from torchft_b200.manager import Manager
from torchft_b200.work import _DummyWork
store = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
dist.init_process_group("gloo", store=dist.PrefixStore("w", store), rank=0, world_size=1)
mesh = init_device_mesh("cpu", (1,))
def mk():
    state = {"step": 0}
    m = create_autospec(Manager, instance=True)
    m._use_async_quorum = False
    m.current_step.side_effect = lambda: state["step"]
    def ar(t, should_quantize=False, reduce_op=None):
        assert not isinstance(t, DTensor); t.mul_(0.5); return _DummyWork(t)
    def ard(out, a, b, should_quantize=False):
        torch.sub(a, b, out=out); return ar(out)
    def commit(): state["step"] += 1; return True
    m.allreduce.side_effect = ar; m.allreduce_delta.side_effect = ard; m.should_commit.side_effect = commit
    return m
def run(shard, flat):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(4, 8), nn.Linear(8, 2))
    if shard:
        for l in model: fully_shard(l, mesh=mesh)
        fully_shard(model, mesh=mesh)
    inner = optim.SGD(model.parameters(), lr=0.1)
    outer = optim.SGD(model.parameters(), lr=0.7, momentum=0.9, nesterov=True)
    g = torch.Generator().manual_seed(1)
    with DiLoCo(mk(), [model], inner, outer, sync_every=3, flat_fragments=flat) as d:
        for _ in range(9):
            inner.zero_grad(); model(torch.randn(5, 4, generator=g)).square().mean().backward(); inner.step()
    return [ (p.to_local() if isinstance(p, DTensor) else p).detach().clone() for p in model.parameters()]
ref = run(False, False)
for flat in (False, None):
    got = run(True, flat)
    for a, b in zip(ref, got): torch.testing.assert_close(a, b)
    print("ok flat=", flat)
# LocalSGD
def run_l(shard):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(4, 8), nn.Linear(8, 2))
    if shard:
        fully_shard(model, mesh=mesh)
    inner = optim.SGD(model.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(1)
    with LocalSGD(mk(), model, inner, sync_every=2):
        for _ in range(6):
            inner.zero_grad(); model(torch.randn(5, 4, generator=g)).square().mean().backward(); inner.step()
    return [ (p.to_local() if isinstance(p, DTensor) else p).detach().clone() for p in model.parameters()]
for a, b in zip(run_l(False), run_l(True)): torch.testing.assert_close(a, b)
print("localsgd ok")
'''
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", child], capture_output=True, text=True, timeout=240, env=dict(os.environ, PYTHONPATH=repo))
    assert r.returncode == 0 and "localsgd ok" in r.stdout and "ok flat= None" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]


def test_diloco_pseudo_gradient_is_what_the_outer_optimizer_sees():
    """At a sync the outer optimizer steps on grad = (last synchronised weights - local weights), averaged by the
    manager, applied to the last synchronised weights (torchft/local_sgd_test.py test_gradient_correctness)."""
    seen = []

    class Recording(optim.SGD):
        def step(self, closure=None):
            seen.append([(p.detach().clone(), p.grad.detach().clone()) for g in self.param_groups for p in g["params"]])
            return super().step(closure)

    torch.manual_seed(0)
    model = TinyModel()
    start = [p.detach().clone() for p in model.parameters()]
    inner = optim.SGD(model.parameters(), lr=0.1)
    outer = Recording(model.parameters(), lr=0.5)
    m = _delta_manager(factor=0.5)
    g = torch.Generator().manual_seed(3)
    with DiLoCo(m, [model], inner, outer, sync_every=2, flat_fragments=False):
        local = None
        for k in range(2):
            inner.zero_grad()
            model(torch.randn(4, 3, generator=g)).square().mean().backward()
            if k == 1:  # what the local weights will be right before the sync
                local = [p.detach() - 0.1 * p.grad for p in model.parameters()]
            inner.step()
    assert len(seen) == 1
    for (p_at_step, grad), s0, l in zip(seen[0], start, local):
        torch.testing.assert_close(p_at_step, s0)               # the outer step starts from the global weights
        torch.testing.assert_close(grad, 0.5 * (s0 - l))         # pseudo-gradient, scaled by the (mock) average
    for p, s0, l in zip(model.parameters(), start, local):
        torch.testing.assert_close(p.detach(), s0 - 0.5 * 0.5 * (s0 - l))


def test_local_sgd_bucketed_average_matches_per_parameter():
    """bucket_cap_mb packs the parameter copies into flat buffers: same averaged weights, fewer collectives."""
    def run(cap_mb):
        torch.manual_seed(0)
        model = TinyModel()
        inner = optim.SGD(model.parameters(), lr=0.1)
        m = mock_manager(commit=True, factor=0.5)
        g = torch.Generator().manual_seed(1)
        with LocalSGD(m, model, inner, sync_every=2, bucket_cap_mb=cap_mb):
            for _ in range(2):
                inner.zero_grad()
                model(torch.randn(4, 3, generator=g)).square().mean().backward()
                inner.step()
        return m.allreduce.call_count, [p.detach().clone() for p in model.parameters()]

    calls_each, each = run(None)
    calls_packed, packed = run(1)
    assert (calls_each, calls_packed) == (4, 1)
    for a, b in zip(each, packed):
        torch.testing.assert_close(a, b)


def test_local_sgd_bucket_cap_splits_and_oversized_parameter():
    big = nn.Linear(600, 600, bias=True)  # weight 1.44 MB > 1 MB cap, bias small
    small = nn.Linear(4, 4)
    model = nn.Sequential(small, big)
    inner = optim.SGD(model.parameters(), lr=0.1)
    m = mock_manager(commit=True, factor=1.0)
    before = [p.detach().clone() for p in model.parameters()]
    LocalSGD(m, model, inner, sync_every=1, bucket_cap_mb=1).sync()
    sizes = sorted(c.args[0].numel() for c in m.allreduce.call_args_list)
    assert sizes == sorted([4 * 4 + 4, 600 * 600, 600])  # small layer together | big weight alone | big bias
    for p, b in zip(model.parameters(), before):
        torch.testing.assert_close(p.detach(), b)
