"""Regression fixtures for DiLoCo: the parameter history of a small seeded model over a grid of
(fragments, sync_every, delay, alpha) is compared with JSON files under ``tests/fixtures/diloco``.
``WRITE_FIXTURE=1 python -m pytest tests/test_diloco_regression.py`` rewrites them after an intended
change of numerics (the reference keeps such fixtures for its mocked-manager DiLoCo runs,
torchft/diloco_regression_test.py:49, test_fixtures/).  Both fragment layouts (per-parameter tensors
and flat buffers with the fused outer step) must follow the same fixture."""

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

FIXTURES = Path(__file__).resolve().parent / "fixtures" / "diloco"
WRITE = os.environ.get("WRITE_FIXTURE", "0") == "1"

GRID = [
    # n_fragments, sync_every, delay, alpha, commit pattern
    (1, 4, 0, 0.0, [True]),
    (2, 4, 0, 0.0, [True]),
    (2, 6, 1, 0.0, [True, True, False]),
    (2, 8, 2, 0.5, [True]),
    (3, 9, 1, 0.25, [True, False, True, True]),
]


def _manager(commit_pattern):
    state = {"step": 0, "votes": 0}
    m = create_autospec(Manager, instance=True)
    m._use_async_quorum = False
    m.current_step.side_effect = lambda: state["step"]

    def allreduce(t, should_quantize=False, reduce_op=None):
        t.mul_(0.5)  # as if a second replica had contributed zeros
        return _DummyWork(t)

    def allreduce_delta(out, a, b, should_quantize=False):
        torch.sub(a, b, out=out)
        return allreduce(out)

    def commit():
        ok = commit_pattern[state["votes"] % len(commit_pattern)]
        state["votes"] += 1
        state["step"] += int(ok)
        return ok

    m.allreduce.side_effect = allreduce
    m.allreduce_delta.side_effect = allreduce_delta
    m.should_commit.side_effect = commit
    return m


def _history(n_frag, sync_every, delay, alpha, pattern, flat):
    torch.manual_seed(1234)
    layers = [nn.Linear(4, 4) for _ in range(n_frag)]
    model = nn.Sequential(*layers)
    inner = optim.AdamW(model.parameters(), lr=5e-2, weight_decay=0.01)
    outers = [optim.SGD(l.parameters(), lr=0.7, momentum=0.9, nesterov=True) for l in layers]
    g = torch.Generator().manual_seed(99)
    hist = []
    with DiLoCo(_manager(pattern), layers, inner, outers, sync_every=sync_every, fragment_sync_delay=delay,
                fragment_update_alpha=alpha, flat_fragments=flat) as d:
        for _ in range(3 * sync_every):
            inner.zero_grad()
            model(torch.randn(8, 4, generator=g)).square().mean().backward()
            inner.step()
            hist.append({
                "local": [round(float(x), 6) for l in layers for x in l.weight.detach().flatten().tolist()],
                "global": [round(float(x), 6) for f in d._fragments for k in sorted(f.original_parameters)
                           for x in f.original_parameters[k].detach().flatten().tolist()],
            })
    return hist


@pytest.mark.parametrize("flat", [False, True])
@pytest.mark.parametrize("n_frag,sync_every,delay,alpha,pattern", GRID)
def test_diloco_history_matches_fixture(n_frag, sync_every, delay, alpha, pattern, flat):
    name = f"f{n_frag}_h{sync_every}_d{delay}_a{alpha}_c{''.join('1' if c else '0' for c in pattern)}.json"
    path = FIXTURES / name
    got = _history(n_frag, sync_every, delay, alpha, pattern, flat)
    if WRITE and not flat:
        path.write_text(json.dumps(got, indent=1) + "\n")
    want = json.loads(path.read_text())
    assert len(got) == len(want)
    for k, (a, b) in enumerate(zip(got, want)):
        assert a["local"] == pytest.approx(b["local"], rel=1e-4, abs=1e-5), (k, a, b)
        assert a["global"] == pytest.approx(b["global"], rel=1e-4, abs=1e-5), (k, a, b)
