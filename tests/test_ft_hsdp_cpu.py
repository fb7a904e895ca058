"""Fault-tolerant HSDP end to end on CPU: two replica groups, each a two-rank gloo job that shards the
Llama trainer's state, gradients averaged across the groups through real Managers and a lighthouse.
Healthy run: both groups end with identical weights.  Recovery: group 1 leaves between steps, is started
again with different weights, heals from group 0 (every rank fetches its own shard from the
same-numbered rank of the healthy group) and ends identical again."""
import json
import os
import socket
import subprocess
import sys
import time

import pytest

from torchft_b200._ftcp import LighthouseServer

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ft_hsdp_cpu_worker.py")


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn_group(group, lighthouse, steps, exit_at=-1, hold=10 ** 9, seed=3, async_quorum=False, diloco=0):
    init_port, store_port = _free_port(), _free_port()
    return [subprocess.Popen(
        [sys.executable, WORKER, "--group", str(group), "--rank", str(r), "--init-port", str(init_port), "--store-port",
         str(store_port), "--lighthouse", lighthouse, "--steps", str(steps), "--exit-at-step", str(exit_at), "--hold-step",
         str(hold), "--seed", str(seed), "--async-quorum", str(int(async_quorum)), "--diloco", str(diloco)],
        stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]


def _results(procs, timeout=240):
    out = []
    for p in procs:
        o, e = p.communicate(timeout=timeout)
        lines = [l for l in o.splitlines() if l.startswith("{")]
        assert p.returncode == 0 and lines, f"rc={p.returncode}\n{o[-1500:]}\n{e[-3000:]}"
        out.append(json.loads(lines[-1]))
    return out


def _assert_same(a, b):
    for x, y in zip(a["unit_sums"], b["unit_sums"]):
        assert abs(x - y) <= 1e-6 * max(1.0, abs(x)), (a["unit_sums"], b["unit_sums"])


def test_ft_hsdp_two_groups_healthy():
    lh = LighthouseServer("[::]:0", 2, join_timeout_ms=500, quorum_tick_ms=20, heartbeat_timeout_ms=2000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    procs = []
    try:
        g0, g1 = _spawn_group(0, addr, 5), _spawn_group(1, addr, 5)
        procs = g0 + g1
        r0, r1 = _results(g0), _results(g1)
        assert all(r["step"] == 5 and r["max_participants"] == 2 and r["errored"] == "None" for r in r0 + r1)
        _assert_same(r0[0], r0[1])
        _assert_same(r0[0], r1[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()


@pytest.mark.parametrize("async_quorum", [False, True])
def test_ft_hsdp_group_leaves_and_heals(async_quorum):
    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=300, quorum_tick_ms=20, heartbeat_timeout_ms=1000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    procs = []
    try:
        g0 = _spawn_group(0, addr, 10, hold=5, async_quorum=async_quorum)
        g1 = _spawn_group(1, addr, 10, exit_at=3, async_quorum=async_quorum)
        procs = g0 + g1
        assert [p.wait(timeout=180) for p in g1] == [17, 17]  # left between steps
        time.sleep(0.5)
        # fresh weights: only healing can make them agree
        g1b = _spawn_group(1, addr, 10, hold=0, seed=99, async_quorum=async_quorum)
        procs += g1b
        r0, r1 = _results(g0), _results(g1b)
        assert r0[0]["step"] == r1[0]["step"] >= 10
        assert all(r["errored"] == "None" and r["max_participants"] == 2 for r in r0 + r1)
        _assert_same(r0[0], r1[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()


def test_engine_diloco_on_sharded_groups():
    """Streaming DiLoCo on the engine with two sharded groups: every rank exchanges the pseudo-gradient of its
    own shard with the same-numbered rank of the other group; after four fragment synchronisations the global
    weights of the two groups are identical."""
    lh = LighthouseServer("[::]:0", 2, join_timeout_ms=500, quorum_tick_ms=20, heartbeat_timeout_ms=2000)
    addr = "http://127.0.0.1:" + lh.address().rsplit(":", 1)[1]
    procs = []
    try:
        g0, g1 = _spawn_group(0, addr, 4, diloco=2), _spawn_group(1, addr, 4, diloco=2)
        procs = g0 + g1
        r0, r1 = _results(g0), _results(g1)
        assert all(r["step"] == 4 and r["commits"] == 4 and r["errored"] == "None" for r in r0 + r1)
        _assert_same(r0[0], r0[1])
        _assert_same(r0[0], r1[0])
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        lh.shutdown()
