"""Control-plane tests: the quorum mathematics on hand-built states (the vectors come from
the behaviour the reference's Rust unit tests pin down, src/lighthouse.rs:627-1112 and
src/manager.rs:880-1107) and end-to-end runs over real sockets in-process."""
import os
import threading
import time
import urllib.request
from datetime import timedelta

import pytest

from torchft_b200 import _ftcp as C

M = C.QuorumMember


def member(rid, step=1, shrink_only=False, commit_failures=0):
    return M(replica_id=rid, address=f"addr_{rid}", store_address=f"store_{rid}", step=step, world_size=1,
             shrink_only=shrink_only, commit_failures=commit_failures)


def quorum_of(ids, qid=1, steps=None):
    q = C.Quorum()
    q.quorum_id = qid
    q.participants = [member(i, step=(steps or {}).get(i, 1)) for i in ids]
    return q


def compute(now, parts, hbs, prev=None, min_replicas=1, join_ms=60000, hb_ms=5000):
    got, reason = C.quorum_compute(now, parts, hbs, prev, min_replicas, join_ms, hb_ms)
    return (None if got is None else [m.replica_id for m in got]), reason


HOUR_MS = 3600 * 1000


def test_quorum_join_timeout():
    now = 1e6
    ids, reason = compute(now, [], {}, join_ms=HOUR_MS)
    assert ids is None
    assert "New quorum not ready, only have 0 participants, need min_replicas 1 [0/0 participants healthy]" in reason
    parts = [(member("a"), now), (member("b"), now)]
    hbs = {"a": now, "b": now}
    assert compute(now, parts, hbs, join_ms=HOUR_MS)[0] == ["a", "b"]
    # a third replica heartbeats but has not joined: wait for it
    hbs["c"] = now
    ids, reason = compute(now, parts, hbs, join_ms=HOUR_MS)
    assert ids is None and "join timeout" in reason
    # ... unless the first joiner has already waited longer than the join timeout
    parts_old = [(member("a"), now - 10 * 3600), (member("b"), now)]
    assert compute(now, parts_old, hbs, join_ms=HOUR_MS)[0] == ["a", "b"]


def test_quorum_heartbeats():
    now = 1e6
    ids, reason = compute(now, [(member("a"), now)], {"a": now - 10}, join_ms=0)
    assert ids is None and "[0/1 participants healthy][0 heartbeating]" in reason
    ids, _ = compute(now, [(member("a"), now), (member("b"), now)], {"a": now - 10, "b": now}, join_ms=0)
    assert ids == ["b"]


def test_quorum_fast_prev_quorum():
    now = 1e6
    prev = quorum_of(["a"])
    # a is back, b heartbeats but has not joined: fast quorum does not wait for b
    ids, reason = compute(now, [(member("a"), now)], {"a": now, "b": now}, prev, join_ms=HOUR_MS)
    assert ids == ["a"] and "Fast quorum" in reason
    # a new joiner rides along
    ids, _ = compute(now, [(member("a"), now), (member("b"), now)], {"a": now, "b": now}, prev, join_ms=HOUR_MS)
    assert ids == ["a", "b"]


def test_quorum_shrink_only():
    now = 1e6
    prev = quorum_of(["a", "b"])
    parts = [(member("a", shrink_only=True), now), (member("c", shrink_only=True), now)]
    ids, reason = compute(now, parts, {"a": now, "c": now}, prev, join_ms=0)
    assert ids == ["a"] and "[shrink_only=true]" in reason


def test_quorum_split_brain():
    now = 1e6
    ids, reason = compute(now, [(member("a"), now)], {"a": now, "b": now}, join_ms=0)
    assert ids is None
    assert "need at least half of 2 healthy workers [1/1 participants healthy][2 heartbeating]" in reason
    ids, _ = compute(now, [(member("a"), now), (member("b"), now)], {"a": now, "b": now, "c": now}, join_ms=0)
    assert ids == ["a", "b"]


def test_quorum_changed():
    a, b = member("1"), member("1")
    assert not C.quorum_changed([a], [b])
    b.address, b.store_address, b.step = "other", "other", 9
    assert not C.quorum_changed([a], [b])
    assert C.quorum_changed([a], [member("2")])
    assert C.quorum_changed([a], [a, member("2")])


def test_compute_quorum_results_first_step():
    q = quorum_of(["replica_0", "replica_1"], qid=1, steps={"replica_0": 0, "replica_1": 0})
    r = C.compute_quorum_results("replica_0", 0, q, True)
    assert (r.heal, r.replica_rank, r.recover_src_replica_rank, r.recover_dst_replica_ranks) == (False, 0, None, [1])
    r = C.compute_quorum_results("replica_1", 0, q, True)
    assert (r.heal, r.replica_rank, r.recover_src_replica_rank, r.recover_dst_replica_ranks) == (True, 1, 0, [])
    assert r.recover_src_manager_address == "addr_replica_0"
    # the primary rotates with the local rank
    r = C.compute_quorum_results("replica_1", 1, q, True)
    assert (r.heal, r.replica_rank, r.recover_dst_replica_ranks) == (False, 1, [0])
    assert r.store_address == "store_replica_1"


def test_compute_quorum_results_recovery():
    steps = {"replica_0": 0, "replica_1": 1, "replica_2": 0, "replica_3": 1, "replica_4": 0}
    q = quorum_of(sorted(steps), qid=1, steps=steps)
    r = C.compute_quorum_results("replica_0", 0, q, True)
    assert r.heal and r.recover_src_replica_rank == 1 and r.recover_src_manager_address == "addr_replica_1"
    assert (r.max_step, r.max_replica_rank, r.max_world_size, r.replica_world_size) == (1, None, 2, 5)
    r = C.compute_quorum_results("replica_1", 0, q, True)
    assert not r.heal and r.recover_dst_replica_ranks == [0, 4] and r.max_replica_rank == 0
    assert r.store_address == "store_replica_1"
    r = C.compute_quorum_results("replica_3", 0, q, True)
    assert not r.heal and r.recover_dst_replica_ranks == [2] and r.max_replica_rank == 1
    # local rank 1 shifts the striping
    r = C.compute_quorum_results("replica_1", 1, q, True)
    assert r.recover_dst_replica_ranks == [2] and r.store_address == "store_replica_3"


def test_compute_quorum_results_skip_init_sync():
    q = quorum_of(["replica_0", "replica_1"], steps={"replica_0": 0, "replica_1": 0})
    assert C.compute_quorum_results("replica_1", 0, q, True).heal
    assert not C.compute_quorum_results("replica_1", 0, q, False).heal
    q = quorum_of(["replica_0", "replica_1"], steps={"replica_0": 1, "replica_1": 0})
    assert C.compute_quorum_results("replica_1", 0, q, False).heal


def test_compute_quorum_results_commit_failures_and_missing():
    q = C.Quorum()
    q.quorum_id = 1
    q.participants = [member("replica_0", 0, commit_failures=0), member("replica_1", 0, commit_failures=2)]
    assert C.compute_quorum_results("replica_0", 0, q, True).commit_failures == 2
    with pytest.raises(RuntimeError, match="not participating"):
        C.compute_quorum_results("nobody", 0, q, True)


# ----------------------------------------------------------------------------- sockets


def test_lighthouse_e2e_and_dashboard():
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10)
    try:
        cl = C.LighthouseClient(lh.address(), timedelta(seconds=5))
        cl.heartbeat("foo")
        q = cl.quorum("foo", timedelta(seconds=5), address="addr", store_address="store", step=10, world_size=1,
                      data={"my_key": "my_value"})
        assert q.quorum_id == 1 and len(q.participants) == 1
        assert q.participants[0].replica_id == "foo" and q.participants[0].step == 10
        assert q.participants[0].data == {"my_key": "my_value"}
        assert q.created.seconds > 0
        port = lh.address().rsplit(":", 1)[1]
        html = urllib.request.urlopen(f"http://localhost:{port}/status", timeout=5).read().decode()
        assert "Previous quorum id: 1" in html and "foo" in html
        index = urllib.request.urlopen(f"http://localhost:{port}/", timeout=5).read().decode()
        assert "Lighthouse Dashboard" in index
    finally:
        lh.shutdown()


def test_lighthouse_join_timeout_bound():
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=400, quorum_tick_ms=10)
    try:
        cl = C.LighthouseClient(lh.address(), timedelta(seconds=5))
        cl.heartbeat("straggler")  # healthy but never joins
        t0 = time.time()
        # split-brain guard: 1 of 2 heartbeating is not a majority until the straggler expires
        with pytest.raises(TimeoutError):
            cl.quorum("a", timedelta(milliseconds=300))
        assert time.time() - t0 < 2.0
    finally:
        lh.shutdown()


def test_lighthouse_heartbeat_expiry_lets_survivor_continue():
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10, heartbeat_timeout_ms=300)
    stop = threading.Event()
    try:
        a = C.LighthouseClient(lh.address(), timedelta(seconds=5))
        b = C.LighthouseClient(lh.address(), timedelta(seconds=5))
        hb = C.LighthouseClient(lh.address(), timedelta(seconds=5))
        a.heartbeat("a")
        b.heartbeat("b")

        def beat():  # what a live manager does every heartbeat interval
            while not stop.is_set():
                hb.heartbeat("a")
                time.sleep(0.05)

        threading.Thread(target=beat, daemon=True).start()
        out = {}
        tb = threading.Thread(target=lambda: out.setdefault("b", b.quorum("b", timedelta(seconds=5))))
        tb.start()
        qa = a.quorum("a", timedelta(seconds=5))
        tb.join()
        assert {p.replica_id for p in qa.participants} == {"a", "b"} and qa.quorum_id == 1
        # b dies (no more heartbeats); a alone gets a new quorum once b's heartbeat expires
        t0 = time.time()
        qa2 = a.quorum("a", timedelta(seconds=5))
        assert [p.replica_id for p in qa2.participants] == ["a"] and qa2.quorum_id == 2
        assert time.time() - t0 < 2.0
    finally:
        stop.set()
        lh.shutdown()


def test_lighthouse_commit_failures_bump_quorum_id():
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10)
    try:
        cl = C.LighthouseClient(lh.address(), timedelta(seconds=5))
        assert cl.quorum("a", timedelta(seconds=5)).quorum_id == 1
        assert cl.quorum("a", timedelta(seconds=5)).quorum_id == 1
    finally:
        lh.shutdown()


def _manager(lh, rid="rep", world_size=1, retries=0):
    return C.ManagerServer(replica_id=rid, lighthouse_addr=lh.address(), hostname="localhost", bind="[::]:0",
                           store_addr="store:1", world_size=world_size, heartbeat_interval=timedelta(milliseconds=50),
                           connect_timeout=timedelta(seconds=5), quorum_retries=retries)


def test_manager_quorum_single_replica():
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10)
    ms = _manager(lh, "rep_id")
    try:
        c = C.ManagerClient(ms.address(), timedelta(seconds=5))
        r = c._quorum(group_rank=0, step=123, checkpoint_metadata="addr", shrink_only=False,
                      timeout=timedelta(seconds=5), init_sync=True, commit_failures=0)
        assert (r.quorum_id, r.max_step, r.max_replica_rank, r.max_world_size) == (1, 123, 0, 1)
        assert (r.replica_rank, r.replica_world_size, r.heal, r.store_address) == (0, 1, False, "store:1")
        assert c._checkpoint_metadata(0, timedelta(seconds=5)) == "addr"
        with pytest.raises(RuntimeError, match="rank not found"):
            c._checkpoint_metadata(7, timedelta(seconds=5))
    finally:
        ms.shutdown()
        lh.shutdown()


def test_manager_should_commit_barrier_and_timeout():
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10)
    ms = _manager(lh, world_size=2)
    try:
        out = {}

        def vote(rank, v):
            c = C.ManagerClient(ms.address(), timedelta(seconds=5))
            out[rank] = c.should_commit(rank, 1, v, timedelta(seconds=5))

        for votes, want in (((True, True), True), ((True, False), False), ((True, True), True)):
            ts = [threading.Thread(target=vote, args=(r, v)) for r, v in enumerate(votes)]
            [t.start() for t in ts]
            [t.join() for t in ts]
            assert out == {0: want, 1: want}
        c = C.ManagerClient(ms.address(), timedelta(seconds=5))
        t0 = time.time()
        with pytest.raises(TimeoutError):
            c.should_commit(0, 2, True, timedelta(milliseconds=100))
        assert time.time() - t0 < 1.0
        # the vote that timed out must not leak into the next round
        ts = [threading.Thread(target=vote, args=(r, True)) for r in range(2)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert out == {0: True, 1: True}
    finally:
        ms.shutdown()
        lh.shutdown()


def test_two_replica_groups_heal_assignment():
    lh = C.LighthouseServer("[::]:0", 2, join_timeout_ms=100, quorum_tick_ms=10)
    m0, m1 = _manager(lh, "rep_0"), _manager(lh, "rep_1")
    try:
        res = {}

        def go(ms, name, step):
            c = C.ManagerClient(ms.address(), timedelta(seconds=5))
            res[name] = c._quorum(group_rank=0, step=step, checkpoint_metadata=name, shrink_only=False,
                                  timeout=timedelta(seconds=5), init_sync=True, commit_failures=0)

        ts = [threading.Thread(target=go, args=(m0, "rep_0", 5)), threading.Thread(target=go, args=(m1, "rep_1", 0))]
        [t.start() for t in ts]
        [t.join() for t in ts]
        a, b = res["rep_0"], res["rep_1"]
        assert a.quorum_id == b.quorum_id == 1
        assert not a.heal and a.recover_dst_replica_ranks == [1] and a.max_replica_rank == 0
        assert b.heal and b.recover_src_replica_rank == 0 and b.recover_src_manager_address == m0.address()
        assert b.max_replica_rank is None and b.max_world_size == 1 and b.replica_world_size == 2
        assert C.ManagerClient(b.recover_src_manager_address, timedelta(seconds=5))._checkpoint_metadata(
            0, timedelta(seconds=5)) == "rep_0"
    finally:
        m0.shutdown()
        m1.shutdown()
        lh.shutdown()


def test_manager_reports_lighthouse_failure_to_all_ranks():
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10)
    ms = _manager(lh, world_size=2, retries=1)
    lh.shutdown()  # lighthouse gone: the round must fail for both ranks, promptly
    try:
        errs = {}

        def go(rank):
            c = C.ManagerClient(ms.address(), timedelta(seconds=5))
            try:
                c._quorum(group_rank=rank, step=0, checkpoint_metadata="", shrink_only=False,
                          timeout=timedelta(seconds=2), init_sync=True, commit_failures=0)
            except (RuntimeError, TimeoutError) as e:
                errs[rank] = e

        t0 = time.time()
        ts = [threading.Thread(target=go, args=(r,)) for r in range(2)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert set(errs) == {0, 1}
        assert time.time() - t0 < 8.0
    finally:
        ms.shutdown()


def test_connect_timeout_raises_timeout_error():
    t0 = time.time()
    with pytest.raises(TimeoutError):
        C.ManagerClient("localhost:1", timedelta(milliseconds=300))
    assert time.time() - t0 < 3.0


def test_lighthouse_join_during_shrink_only_round():
    """A replica that asks to join while the others shrink waits through the shrink-only round and
    is admitted in the next one: participant counts 2, 2, 3 (src/lighthouse.rs:1114-1225)."""
    lh = C.LighthouseServer("[::]:0", 2, join_timeout_ms=100, quorum_tick_ms=10)
    try:
        clients = {r: C.LighthouseClient(lh.address(), timedelta(seconds=5)) for r in "abc"}

        def ask(rid, out, **kw):
            out[rid] = clients[rid].quorum(rid, timedelta(seconds=10), **kw)

        def round_(specs):
            out, threads = {}, []
            for rid, kw in specs.items():
                t = threading.Thread(target=ask, args=(rid, out), kwargs=kw)
                t.start()
                threads.append(t)
            return out, threads

        out1, th = round_({"a": {}, "b": {}})
        for t in th:
            t.join()
        assert {len(q.participants) for q in out1.values()} == {2}
        # a and b shrink; c asks to join in the same round and has to wait
        out2, th2 = round_({"a": {"shrink_only": True}, "b": {"shrink_only": True}})
        joiner_out = {}
        tc = threading.Thread(target=ask, args=("c", joiner_out))
        tc.start()
        for t in th2:
            t.join()
        assert all(sorted(p.replica_id for p in q.participants) == ["a", "b"] for q in out2.values())
        assert "c" not in joiner_out  # still blocked
        out3, th3 = round_({"a": {}, "b": {}})
        for t in th3:
            t.join()
        tc.join()
        assert all(len(q.participants) == 3 for q in list(out3.values()) + [joiner_out["c"]])
    finally:
        lh.shutdown()


def test_commit_failures_reported_by_a_member_bump_the_quorum_id():
    """Same membership, but a member reports failed commits: the lighthouse issues a new quorum id so
    that every group reconfigures its process group (src/lighthouse.rs:1263-1293)."""
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10)
    mgr = _manager(lh)
    try:
        cl = C.ManagerClient(mgr.address(), timedelta(seconds=5))
        ids = []
        for failures in (0, 0, 2, 0):
            r = cl._quorum(group_rank=0, step=1, checkpoint_metadata="m", shrink_only=False, timeout=timedelta(seconds=5),
                           init_sync=False, commit_failures=failures)
            ids.append((r.quorum_id, r.commit_failures))
        assert ids[0][0] == ids[1][0]
        assert ids[2][0] == ids[1][0] + 1 and ids[2][1] == 2
        assert ids[3][0] == ids[2][0]
    finally:
        mgr.shutdown()
        lh.shutdown()


def test_manager_retries_until_the_lighthouse_answers():
    """The lighthouse goes away and comes back on the same port while a quorum request is in flight:
    with quorum_retries the manager reconnects and the request succeeds (the role MockLighthouse plays
    in src/manager.rs:1109-1217)."""
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10)
    port = lh.address().rsplit(":", 1)[1]
    ms = C.ManagerServer(replica_id="late", lighthouse_addr=lh.address(), hostname="localhost", bind="[::]:0",
                         store_addr="store:1", world_size=1, heartbeat_interval=timedelta(milliseconds=50),
                         connect_timeout=timedelta(seconds=1), quorum_retries=8)
    try:
        c = C.ManagerClient(ms.address(), timedelta(seconds=5))
        first = c._quorum(group_rank=0, step=4, checkpoint_metadata="m", shrink_only=False, timeout=timedelta(seconds=10),
                          init_sync=False, commit_failures=0)
        assert first.max_step == 4
        lh.shutdown()
        lh = None
        out = {}

        def ask():
            out["r"] = c._quorum(group_rank=0, step=5, checkpoint_metadata="m", shrink_only=False,
                                 timeout=timedelta(seconds=30), init_sync=False, commit_failures=0)

        t = threading.Thread(target=ask)
        t.start()
        time.sleep(0.5)  # the first attempts fail: nothing listens
        lh = C.LighthouseServer(f"[::]:{port}", 1, join_timeout_ms=100, quorum_tick_ms=10)
        t.join(30)
        assert not t.is_alive() and out["r"].max_step == 5 and out["r"].replica_world_size == 1
    finally:
        ms.shutdown()
        if lh is not None:
            lh.shutdown()


def test_should_commit_declines_when_ranks_vote_for_different_steps():
    """Two ranks of one group that drifted to different steps must not commit together (the reference's
    barrier ignores `step`); the round after, with matching steps, commits again."""
    lh = C.LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10)
    ms = _manager(lh, world_size=2)
    try:
        def vote(rank, step, out):
            c = C.ManagerClient(ms.address(), timedelta(seconds=5))
            out[rank] = c.should_commit(rank, step, True, timedelta(seconds=5))

        for steps, want in (((7, 8), False), ((9, 9), True)):
            out = {}
            ts = [threading.Thread(target=vote, args=(r, steps[r], out)) for r in range(2)]
            for t in ts:
                t.start()
            for t in ts:
                t.join()
            assert out == {0: want, 1: want}, (steps, out)
    finally:
        ms.shutdown()
        lh.shutdown()


def test_control_plane_threads_are_named():
    """Server threads carry names (visible in ps -L / top -H / debuggers), as the reference names its runtime
    threads torchft-lighths / torchft-manager (src/lib.rs:105,337)."""
    import os
    import time as _time
    from datetime import timedelta as _td

    from torchft_b200.coordination import LighthouseServer, ManagerServer

    def names():
        out = []
        for t in os.listdir("/proc/self/task"):
            try:
                out.append(open(f"/proc/self/task/{t}/comm").read().strip())
            except OSError:
                pass
        return out

    lh = LighthouseServer(bind="[::]:0", min_replicas=1)
    ms = ManagerServer(replica_id="named", lighthouse_addr=lh.address(), hostname="localhost", bind="[::]:0",
                       store_addr="localhost:1", world_size=1, heartbeat_interval=_td(milliseconds=50),
                       connect_timeout=_td(seconds=5))
    try:
        _time.sleep(0.3)
        got = names()
        for want in ("ftb-lighths-acc", "ftb-lighths-tic", "ftb-manager-acc", "ftb-manager-hb", "ftb-lighths-con"):
            assert want in got, (want, got)
    finally:
        ms.shutdown()
        lh.shutdown()


def test_dashboard_kill_button_ends_the_replica_process():
    """POST /replica/<id>/kill on the lighthouse reaches the replica's manager server, which exits the
    process with status 1 (src/lighthouse.rs:454-479, src/manager.rs:481-486); an unknown id is an error."""
    import subprocess
    import sys
    import urllib.error
    import urllib.parse
    import urllib.request

    from torchft_b200.coordination import LighthouseServer

    lh = LighthouseServer(bind="[::]:0", min_replicas=1, join_timeout_ms=100)
    port = lh.address().rsplit(":", 1)[1]
    base = f"http://127.0.0.1:{port}"
    child = f'''
import time
from datetime import timedelta
from torchft_b200.coordination import ManagerClient, ManagerServer
ms = ManagerServer(replica_id="victim:1", lighthouse_addr="{base}", hostname="127.0.0.1", bind="[::]:0",
                   store_addr="127.0.0.1:1", world_size=1, heartbeat_interval=timedelta(milliseconds=50),
                   connect_timeout=timedelta(seconds=5))
c = ManagerClient(ms.address(), timedelta(seconds=5))
c._quorum(group_rank=0, step=0, checkpoint_metadata="", shrink_only=False, timeout=timedelta(seconds=10),
          init_sync=False, commit_failures=0)
print("joined", flush=True)
time.sleep(60)
'''
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.Popen([sys.executable, "-c", child], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         env=dict(os.environ, PYTHONPATH=repo))
    try:
        assert p.stdout.readline().strip() == "joined"
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(urllib.request.Request(f"{base}/replica/nobody/kill", method="POST"), timeout=5)
        assert e.value.code == 500
        assert p.poll() is None
        url = f"{base}/replica/{urllib.parse.quote('victim:1', safe='')}/kill"
        assert urllib.request.urlopen(urllib.request.Request(url, method="POST"), timeout=15).read() == b"ok"
        assert p.wait(timeout=15) == 1
    finally:
        if p.poll() is None:
            p.kill()
        lh.shutdown()


def test_servers_survive_malformed_input():
    """Garbage, truncated frames, oversized length fields and random bodies for every method id leave the
    lighthouse and a manager server running and still answering.  In a child process: a crash of the native
    code must fail this test, not the test runner."""
    import subprocess
    import sys

    child = r'''
import os, random, socket, struct, time
from datetime import timedelta
from torchft_b200.coordination import LighthouseServer, ManagerClient, ManagerServer

lh = LighthouseServer(bind="[::]:0", min_replicas=1, join_timeout_ms=50, heartbeat_timeout_ms=300)
lport = int(lh.address().rsplit(":", 1)[1])
ms = ManagerServer(replica_id="fuzz", lighthouse_addr=f"http://127.0.0.1:{lport}", hostname="127.0.0.1", bind="[::]:0",
                   store_addr="127.0.0.1:1", world_size=1, heartbeat_interval=timedelta(milliseconds=50),
                   connect_timeout=timedelta(seconds=5))
mport = int(ms.address().rsplit(":", 1)[1])
rnd = random.Random(1234)

def poke(port, payload, linger=0.02):
    s = socket.create_connection(("127.0.0.1", port), timeout=2)
    try:
        s.sendall(payload)
        s.settimeout(linger)
        try:
            s.recv(4096)
        except (socket.timeout, ConnectionError):
            pass
    finally:
        s.close()

def frame(method, body, timeout_ms=50, length=None):
    return b"FTB2" + struct.pack("<IBQ", len(body) if length is None else length, method, timeout_ms) + body

cases = 0
for port in (lport, mport):
    poke(port, b"")                                        # connect and leave
    poke(port, os.urandom(3))                              # less than a magic
    poke(port, os.urandom(64))                             # garbage (treated as a broken HTTP request)
    poke(port, b"FTB2" + os.urandom(5))                    # truncated header
    poke(port, frame(1, b"", length=0xFFFFFFFF))           # absurd length field
    poke(port, frame(1, b"abc", length=1 << 20))           # body shorter than announced
    poke(port, b"GET /" + b"a" * 70000 + b" HTTP/1.1\r\n\r\n")   # oversized request line
    poke(port, b"POST /replica/%zz/kill HTTP/1.1\r\nContent-Length: 99999999999\r\n\r\n")
    for method in range(0, 12):
        for _ in range(12):
            n = rnd.choice([0, 1, 2, 7, 33, 200, 4096])
            poke(port, frame(method, bytes(rnd.getrandbits(8) for _ in range(n))))
            cases += 1
    # valid prefix of a real message, cut at every length
    good = b"\x0a\x05hello\x10\x01\x18\x02\x22\x03abc"
    for cut in range(len(good)):
        poke(port, frame(1, good[:cut]))
        poke(port, frame(2, good[:cut]))

# Random bodies that happen to decode as heartbeats or quorum requests register phantom replicas (the protocol has no
# authentication); they stop counting once their heartbeats are older than the timeout.
time.sleep(0.6)
# both servers still work: the manager's quorum goes through the lighthouse
r = ManagerClient(ms.address(), timedelta(seconds=5))._quorum(group_rank=0, step=0, checkpoint_metadata="", shrink_only=False,
        timeout=timedelta(seconds=10), init_sync=False, commit_failures=0)
assert r.replica_world_size == 1 and r.quorum_id >= 1
ms.shutdown(); lh.shutdown()
print("survived", cases)
'''
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", child], capture_output=True, text=True, timeout=280, env=dict(os.environ, PYTHONPATH=repo))
    assert r.returncode == 0 and "survived" in r.stdout, f"rc={r.returncode}\n{r.stdout[-1500:]}\n{r.stderr[-3000:]}"


def test_lighthouse_metrics_endpoint():
    """GET /metrics: Prometheus text exposition of the quorum state (an addition; the reference exposes no metrics)."""
    from torchft_b200.coordination import LighthouseClient, LighthouseServer

    lh = LighthouseServer(bind="[::]:0", min_replicas=1, join_timeout_ms=50)
    try:
        port = lh.address().rsplit(":", 1)[1]
        cl = LighthouseClient(f"http://127.0.0.1:{port}", timedelta(seconds=5))
        cl.quorum(replica_id="m0", timeout=timedelta(seconds=5), step=7)
        cl.heartbeat('odd"name')  # afterwards: a second heartbeating replica that never joins would block the quorum
        text = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5).read().decode()
        values = {}
        for line in text.splitlines():
            if line and not line.startswith("#"):
                name, value = line.rsplit(" ", 1)
                values[name] = float(value)
        assert values["torchft_lighthouse_quorum_id"] == 1
        assert values["torchft_lighthouse_quorum_participants"] == 1
        assert values["torchft_lighthouse_quorums_issued_total"] == 1
        assert values["torchft_lighthouse_quorum_requests_total"] == 1
        assert values["torchft_lighthouse_heartbeats_total"] == 1
        assert values["torchft_lighthouse_healthy_replicas"] == 2
        assert values['torchft_lighthouse_replica_step{replica="m0"}'] == 7
        assert values['torchft_lighthouse_heartbeat_age_seconds{replica="odd\\"name"}'] < 5
        assert "# TYPE torchft_lighthouse_quorums_issued_total counter" in text
    finally:
        lh.shutdown()
