"""Stock PyTorch FSDP2 inside each replica group + the managed replicate dimension, end to end on CPU: two
groups of two gloo ranks, real Managers and a lighthouse.  The groups start from different weights (the first
quorum's init_sync heals group 1's shards from group 0), train on different data and must end identical,
rank by rank.  Then a group leaves between steps, restarts with other weights and heals."""
import json
import os
import socket
import subprocess
import sys
import time

import pytest

from torchft_b200._ftcp import LighthouseServer

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_fsdp_ft_worker.py")


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn_group(group, lighthouse, steps, exit_at=-1, seed=0, hold=10 ** 9):
    init_port, store_port = _free_port(), _free_port()
    env = dict(os.environ, OMP_NUM_THREADS="1")
    return [subprocess.Popen(
        [sys.executable, WORKER, "--group", str(group), "--rank", str(r), "--init-port", str(init_port), "--store-port",
         str(store_port), "--lighthouse", lighthouse, "--steps", str(steps), "--exit-at-step", str(exit_at), "--seed", str(seed),
         "--hold-step", str(hold)],
        stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env) for r in range(2)]


def _results(procs, timeout=240):
    out = []
    for p in procs:
        o, e = p.communicate(timeout=timeout)
        lines = [l for l in o.splitlines() if l.startswith("{")]
        assert p.returncode == 0 and lines, f"rc={p.returncode}\n{o[-1500:]}\n{e[-3000:]}"
        out.append(json.loads(lines[-1]))
    return out


def _assert_same(a, b):
    for x, y in zip(a["sums"], b["sums"]):
        assert abs(x - y) <= 1e-5 * max(1.0, abs(x)), (a["sums"], b["sums"])


def _single_process_reference(steps):
    """The same model, data and optimizer as tests/_fsdp_ft_worker.py without any parallelism: the mean gradient over
    the batches of all (group, rank) pairs, SGD with momentum.  Initial weights are what init_sync leaves behind: the
    recovery source rotates with the rank inside the group, so rank 0's shards (the first half of every parameter's
    rows) are group 0's initial values and rank 1's shards are group 1's."""
    import torch
    from torch import nn

    def init(seed):
        torch.manual_seed(seed)
        return nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 8))

    model, other = init(100), init(101)
    with torch.no_grad():
        for p, q in zip(model.parameters(), other.parameters()):
            half = p.shape[0] // 2
            p[half:].copy_(q[half:])
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    for step in range(steps):
        opt.zero_grad()
        for group in range(2):
            for rank in range(2):
                g = torch.Generator().manual_seed(1000 * group + 10 * rank + step)
                x, y = torch.randn(8, 16, generator=g), torch.randn(8, 8, generator=g)
                ((model(x) - y).square().mean() / 4).backward()
        opt.step()
    return [p.detach() for p in model.parameters()]


@pytest.mark.timeout(400)
def test_fsdp2_groups_agree_after_init_sync_and_training():
    lh = LighthouseServer("[::]:0", 2, join_timeout_ms=500, quorum_tick_ms=20, heartbeat_timeout_ms=2000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    procs = []
    try:
        g0, g1 = _spawn_group(0, addr, 5, seed=0), _spawn_group(1, addr, 5, seed=1)
        procs = g0 + g1
        r0, r1 = _results(g0), _results(g1)
        assert all(r["step"] == 5 and r["participants"] == 2 for r in r0 + r1)
        assert all(r["batches"] == 10 for r in r0 + r1)
        for rank in range(2):  # same-numbered ranks hold the same shards
            _assert_same(r0[rank], r1[rank])
        assert r0[0]["sums"] != r0[1]["sums"]  # the two ranks of a group hold different shards
        # and the shards are those of plain single-process training on the union of the four ranks' batches: the
        # reduce-scatter inside a group and the managed all-reduce across groups together form the global mean gradient
        want = _single_process_reference(steps=5)
        for rank in range(2):
            for got, full in zip(r0[rank]["sums"], want):
                shard = full.chunk(2, dim=0)[rank]
                assert abs(got - float(shard.double().sum())) <= 1e-4 * max(1.0, abs(got)), (rank, got, float(shard.double().sum()))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()


@pytest.mark.timeout(600)
def test_fsdp2_group_leaves_and_heals():
    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=300, quorum_tick_ms=20, heartbeat_timeout_ms=1000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    procs = []
    try:
        g0 = _spawn_group(0, addr, 10, seed=0, hold=5)
        g1 = _spawn_group(1, addr, 10, exit_at=3, seed=1)
        procs = g0 + g1
        assert [p.wait(timeout=180) for p in g1] == [17, 17]
        time.sleep(0.5)
        g1b = _spawn_group(1, addr, 10, seed=7, hold=0)
        procs += g1b
        r0, r1 = _results(g0), _results(g1b)
        assert r0[0]["step"] == r1[0]["step"] >= 10
        assert all(r["participants"] == 2 for r in r0 + r1)
        assert r1[0]["batches"] == r0[0]["batches"] > r0[0]["step"]  # counters healed too; some steps had two groups
        for rank in range(2):
            _assert_same(r0[rank], r1[rank])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()
