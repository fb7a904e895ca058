"""DiLoCo against the reference's own golden histories.

The reference ships the parameter histories of its mocked-update DiLoCo runs (1x1 weights starting at 1,
constant gradient 2, inner step ``p -= 1 * grad``, outer step ``p -= 2 * pseudo_gradient``, ``sync_every`` 6,
two fragments; torchft/diloco_regression_test.py:289-375, files under ``test_fixtures/``).  Both of its
replicas hold the same numbers, so the average of their pseudo-gradients is the pseudo-gradient itself and a
manager whose allreduce is the identity reproduces the run.  The per-parameter fragments (with the
reference's plain-update outer optimizer) and the flat fragments (``torch.optim.SGD(lr=2)``, the same update)
must both follow those files step by step.  The files are read from the reference checkout when it is present
(they are data of the reference, not part of this repository); without it the test is skipped.
"""
import json
import os
from pathlib import Path
from unittest.mock import create_autospec

import pytest
import torch
from torch import nn, optim

from torchft_b200.local_sgd import DiLoCo
from torchft_b200.manager import Manager
from torchft_b200.work import _DummyWork

_REPO = Path(__file__).resolve().parent.parent
# the reference's golden histories: in the plain copy of the reference that the benchmarks' reference arm uses, or in
# a checkout of the reference named by TORCHFT_REFERENCE
_DIRS = [_REPO / "baseline" / "_ref" / "test_fixtures"]
if os.environ.get("TORCHFT_REFERENCE"):
    _DIRS.insert(0, Path(os.environ["TORCHFT_REFERENCE"]) / "test_fixtures")
_NAME = "torchft.diloco_regression_test.DiLoCoMockedUpdateTest.test_diloco_mocked_updates_{}.json"
# the order of the reference's parameter grid: (fragment_sync_delay, fragment_update_alpha)
CASES = [(0, 0.0), (0, 0.5), (0, 1.0), (1, 0.0), (1, 0.5), (1, 1.0)]


def _fixture(i):
    for d in _DIRS:
        p = d / _NAME.format(i)
        if p.is_file():
            return json.loads(p.read_text())
    pytest.skip("the reference's test_fixtures are not on this machine")


class _PlainUpdate(optim.Optimizer):
    """p -= lr * grad, the reference's mock optimizer."""

    def __init__(self, params, lr):
        super().__init__(params, dict(lr=lr))

    def step(self, closure=None):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    p.data.add_(p.grad.data, alpha=-g["lr"])


def _manager():
    state = {"step": 0}
    m = create_autospec(Manager, instance=True)
    m._use_async_quorum = False
    m.current_step.side_effect = lambda: state["step"]
    m.allreduce.side_effect = lambda t, should_quantize=False, reduce_op=None: _DummyWork(t)

    def allreduce_delta(out, a, b, should_quantize=False):
        torch.sub(a, b, out=out)
        return _DummyWork(out)

    def commit():
        state["step"] += 1
        return True

    m.allreduce_delta.side_effect = allreduce_delta
    m.should_commit.side_effect = commit
    return m


def _run(delay, alpha, flat):
    layers = nn.ModuleList([nn.Linear(1, 1, bias=False) for _ in range(2)])
    with torch.no_grad():
        for l in layers:
            l.weight.fill_(1.0)
    inner = _PlainUpdate(layers.parameters(), lr=1.0)
    if flat:
        outers = [optim.SGD(l.parameters(), lr=2.0) for l in layers]
    else:
        outers = [_PlainUpdate(l.parameters(), lr=2.0) for l in layers]
    m = _manager()
    history, global_history, seen = {}, {}, set()
    with DiLoCo(m, list(layers), inner, outers, sync_every=6, backup_device=torch.device("cpu"),
                fragment_sync_delay=delay, fragment_update_alpha=alpha, flat_fragments=flat) as d:
        assert d.flat_fragments == flat
        local_step = 0
        while True:
            history[str(local_step)] = {f"layers.{i}.weight": l.weight.detach().tolist() for i, l in enumerate(layers)}
            step = m.current_step()
            if step == 5:  # five synchronisations, as far as the reference histories go
                break
            if step not in seen:
                seen.add(step)
                global_history[str(local_step)] = {
                    f"layers.{i}.weight": f.original_parameters["weight"].detach().tolist() for i, f in enumerate(d._fragments)}
            for l in layers:
                l.weight.grad = torch.full_like(l.weight, 2.0)
            inner.step()
            local_step += 1
    return history, global_history


@pytest.mark.parametrize("flat", [False, True])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_history_follows_the_reference_fixture(case, flat):
    want = _fixture(case)[0][0]  # replica 0 (both replicas hold the same numbers)
    delay, alpha = CASES[case]
    history, global_history = _run(delay, alpha, flat)
    assert set(history) == set(want["history"])
    for k, params in want["history"].items():
        for name, v in params.items():
            assert history[k][name][0] == pytest.approx(v[0], rel=1e-5, abs=1e-5), (k, name)
    assert set(global_history) == set(want["global_parameter_history"])
    for k, params in want["global_parameter_history"].items():
        for name, v in params.items():
            assert global_history[k][name][0] == pytest.approx(v[0], rel=1e-5, abs=1e-5), (k, name)
