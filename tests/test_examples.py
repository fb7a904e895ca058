"""The example trainers run as a user would start them: a lighthouse, then one ``torchrun`` per
replica group (train_ddp.py / train_diloco.py in the reference are started the same way,
README.md "Example Training Loop (DDP)").  CPU, Gloo."""

import os
import random
import socket
import subprocess
import sys
import threading
import time
from pathlib import Path

import psutil
import pytest

from torchft_b200.coordination import LighthouseServer

REPO = Path(__file__).resolve().parent.parent


def _free_port_pair() -> int:
    """A port P below the ephemeral range such that P and P+1 can both be bound right now (the runner gives group g
    the port base+g; ports inside the ephemeral range can be taken by an outgoing connection at any moment)."""
    rnd = random.Random(os.getpid() ^ int(time.time() * 1000))
    for _ in range(200):
        p = rnd.randrange(20000, 30000, 2)
        try:
            with socket.socket() as a, socket.socket() as b:
                a.bind(("127.0.0.1", p))
                b.bind(("127.0.0.1", p + 1))
            return p
        except OSError:
            continue
    raise RuntimeError("no free port pair found")


def _launch(script: str, group: int, lighthouse: str, port: int = 0, **env) -> subprocess.Popen:
    port = port or _free_port_pair()
    full = dict(os.environ, TORCHFT_LIGHTHOUSE=lighthouse, REPLICA_GROUP_ID=str(group), NUM_REPLICA_GROUPS="2",
                PYTHONPATH=str(REPO), OMP_NUM_THREADS="2", **env)  # two trainers share the cores: no oversubscription
    return subprocess.Popen(
        [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nproc-per-node", "1",
         "--master-port", str(port), str(REPO / script)],
        env=full, cwd=REPO, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)


def _kill_tree(pid: int) -> None:
    """SIGKILL a launcher and everything it started.  torchrun puts its workers into sessions of their own,
    so the launcher's process group does not reach them; the children are looked up by pid instead."""
    try:
        root = psutil.Process(pid)
    except psutil.NoSuchProcess:
        return
    procs = root.children(recursive=True) + [root]
    for q in procs:
        try:
            q.kill()
        except psutil.NoSuchProcess:
            pass
    psutil.wait_procs(procs, timeout=10)


def _finish(p: subprocess.Popen, timeout: float = 240) -> str:
    try:
        out, _ = p.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        _kill_tree(p.pid)
        out, _ = p.communicate()
        pytest.fail("example did not finish:\n" + out[-3000:])
    return out


@pytest.mark.timeout(600)
def test_train_ddp_two_groups_cpu():
    lh = LighthouseServer(bind="[::]:0", min_replicas=1, join_timeout_ms=1000)
    try:
        procs = [_launch("train_ddp.py", g, lh.address(), STEPS="6") for g in range(2)]
        outs = [_finish(p) for p in procs]
        for p, out in zip(procs, outs):
            assert p.returncode == 0, out[-3000:]
            assert "step 5] should_commit=True" in out, out[-3000:]
    finally:
        lh.shutdown()


class _Tail:
    """Collects a process's output on a thread so that a test can wait for a line to appear."""

    def __init__(self, p: subprocess.Popen) -> None:
        self.p, self.lines, self._lock = p, [], threading.Lock()
        self._t = threading.Thread(target=self._pump, daemon=True)
        self._t.start()

    def _pump(self) -> None:
        for line in self.p.stdout:
            with self._lock:
                self.lines.append(line)

    def text(self) -> str:
        with self._lock:
            return "".join(self.lines)

    def wait_for_count(self, needle: str, count: int, timeout: float) -> None:
        end = time.monotonic() + timeout
        while self.text().count(needle) < count:
            if time.monotonic() > end or self.p.poll() is not None:
                pytest.fail(f"{needle!r} did not appear {count} times:\n" + self.text()[-3000:])
            time.sleep(0.2)

    def finish(self, timeout: float) -> str:
        try:
            self.p.wait(timeout)
        except subprocess.TimeoutExpired:
            _kill_tree(self.p.pid)
            self.p.wait()
            pytest.fail("example did not finish:\n" + self.text()[-3000:])
        self._t.join(10)
        return self.text()


@pytest.mark.timeout(900)
def test_train_ddp_restarted_group_heals_cpu():
    """Group 1 is killed mid-run and started again: it rejoins, copies the state from group 0 and both
    reach the last step; group 0 never stops."""
    lh = LighthouseServer(bind="[::]:0", min_replicas=1, join_timeout_ms=1000, heartbeat_timeout_ms=1000)
    steps = 2500  # the survivor must still be training when the restarted group is back
    t0 = t1 = t1b = None
    try:
        t0 = _Tail(_launch("train_ddp.py", 0, lh.address(), STEPS=str(steps)))
        t1 = _Tail(_launch("train_ddp.py", 1, lh.address(), STEPS=str(steps)))
        t1.wait_for_count("should_commit=True", 20, 120)  # (it may have healed past any particular step number)
        _kill_tree(t1.p.pid)
        t1.p.wait()
        t1b = _Tail(_launch("train_ddp.py", 1, lh.address(), STEPS=str(steps)))
        out0, out1 = t0.finish(600), t1b.finish(600)
        assert t0.p.returncode == 0, out0[-3000:]
        assert t1b.p.returncode == 0, out1[-3000:]
        last = f"step {steps - 1}] should_commit=True"
        assert last in out0 and last in out1
        # the restarted group did not start from step 0: it healed to the survivor's step
        assert "healing required" in out1, out1[:3000]
        assert "step 1] should_commit" not in out1
        assert "peers need recovery from us" in out0
    finally:
        for t in (t0, t1, t1b):
            if t is not None:
                _kill_tree(t.p.pid)
        lh.shutdown()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("streaming", ["0", "1"])
def test_train_diloco_two_groups_cpu(streaming):
    lh = LighthouseServer(bind="[::]:0", min_replicas=1, join_timeout_ms=1000)
    try:
        procs = [_launch("train_diloco.py", g, lh.address(), STEPS="45", USE_STREAMING=streaming)
                 for g in range(2)]
        outs = [_finish(p) for p in procs]
        for p, out in zip(procs, outs):
            assert p.returncode == 0, out[-3000:]
            assert "should_commit=True" in out and "local_step=40" in out, out[-3000:]
    finally:
        lh.shutdown()


@pytest.mark.timeout(900)
def test_runner_and_punisher_with_real_trainers(tmp_path):
    """The job runner supervises two real train_ddp.py groups; the punisher injects a communication failure
    (the process survives, the step is discarded, the group is rebuilt), then kills a group (every process of
    it, no orphaned trainer stays in the job), which the runner restarts; both groups finish."""
    from torchft_b200.launch.runner import Punisher, Runner, _descendants

    pid_file, logs = str(tmp_path / "pids.json"), tmp_path / "logs"
    steps = 3000  # long enough that group 0 is still training when the killed group is back, even on a loaded host
    runner = Runner([str(REPO / "train_ddp.py")], num_groups=2, base_port=_free_port_pair(), max_restarts=3, pid_file=pid_file,
                    poll_secs=0.2, log_dir=str(logs), extra_env={"STEPS": str(steps), "OMP_NUM_THREADS": "2", "PYTHONPATH": str(REPO)})
    result = {}
    th = threading.Thread(target=lambda: result.setdefault("rc", runner.run()), daemon=True)
    th.start()

    def log(g, restart=0):
        f = logs / f"group_{g}.{restart}.log"
        return f.read_text() if f.exists() else ""

    def wait(cond, timeout, what):
        end = time.monotonic() + timeout
        while not cond():
            assert time.monotonic() < end and th.is_alive(), f"{what}:\n{log(0)[-1500:]}\n{log(1)[-1500:]}"
            time.sleep(0.2)

    try:
        wait(lambda: log(0).count("should_commit=True") > 20 and log(1).count("should_commit=True") > 20, 180, "never stepped")
        pun = Punisher(pid_file)
        assert pun.inject("comms", group=1) == 1
        wait(lambda: "injected communication failure" in log(1), 30, "no injection seen")
        before = log(1).count("should_commit=True")
        wait(lambda: log(1).count("should_commit=True") > before + 20, 120, "group 1 did not recover from the comms fault")
        assert "should_commit=False" in log(1)
        assert not (logs / "group_1.1.log").exists()  # it was never restarted: the process survived

        with open(pid_file) as f:
            import json
            launcher = json.load(f)["1"]
        victims = [launcher] + _descendants(launcher)
        assert len(victims) >= 2
        assert pun.inject("kill", group=1) == 1
        wait(lambda: all(not os.path.exists(f"/proc/{q}") or open(f"/proc/{q}/stat").read().split(")")[-1].split()[0] == "Z"
                         for q in victims), 30, "killed group left processes behind")
        wait(lambda: "healing required" in log(1, 1), 180, "restarted group did not heal")
        th.join(600)
        assert not th.is_alive() and result.get("rc") == 0, (result, log(0)[-1500:], log(1, 1)[-1500:])
        assert f"step {steps - 1}] should_commit=True" in log(0)
        assert f"step {steps - 1}] should_commit=True" in log(1, 1)
        assert "participants=3" not in log(0)  # the dead group's trainer did not linger as a third replica
        with pytest.raises(ValueError):
            pun.inject("meteor")
    finally:
        for gp in runner._groups:
            if gp.proc is not None:
                _kill_tree(gp.proc.pid)


@pytest.mark.timeout(600)
def test_train_hsdp_cpu_with_durable_checkpoint_resume(tmp_path):
    """train_hsdp.py on CPU (Gloo): two replica groups of two shard ranks under one torchrun; the job writes durable
    checkpoints, is started again and resumes from the newest complete one."""
    ckpt = tmp_path / "ckpt"

    def run(steps):
        port = _free_port_pair()
        env = dict(os.environ, PYTHONPATH=str(REPO), OMP_NUM_THREADS="1")
        return subprocess.run(
            [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr", "127.0.0.1",
             "--master-port", str(port), str(REPO / "train_hsdp.py"), "--model", "llama-tiny", "--seq-len", "16", "--steps", str(steps),
             "--replica-groups", "2", "--ckpt-dir", str(ckpt), "--ckpt-every", "5"],
            cwd=REPO, env=env, capture_output=True, text=True, timeout=280)

    r = run(10)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "participants 2" in r.stdout
    done = sorted(p.name for p in ckpt.iterdir())
    assert "step_00000010" in done and all((ckpt / "step_00000010" / f"rank_{k}.pt").is_file() for k in range(2))
    r = run(15)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "resumed from step 10" in r.stdout and "step 10 loss" in r.stdout and "step 0 loss" not in r.stdout


@pytest.mark.timeout(600)
def test_runner_detects_a_hung_group(tmp_path, capfd):
    """A trainer that is alive but stuck (SIGSTOP here) stops voting on commits; the runner notices through the
    managers' progress files, kills the group's processes and starts it again."""
    import signal

    from torchft_b200.launch.runner import Runner, _descendants

    logs = tmp_path / "logs"
    runner = Runner([str(REPO / "train_ddp.py")], num_groups=1, base_port=_free_port_pair(), max_restarts=2,
                    pid_file=str(tmp_path / "pids.json"), poll_secs=0.2, log_dir=str(logs), hang_timeout_secs=12.0,
                    progress_dir=str(tmp_path / "progress"),
                    extra_env={"STEPS": "800", "OMP_NUM_THREADS": "2", "PYTHONPATH": str(REPO)})
    result = {}
    th = threading.Thread(target=lambda: result.setdefault("rc", runner.run()), daemon=True)
    th.start()
    try:
        first = logs / "group_0.0.log"
        end = time.monotonic() + 120
        while not (first.exists() and first.read_text().count("should_commit=True") > 10):
            assert time.monotonic() < end and th.is_alive(), first.read_text()[-1500:] if first.exists() else "no log"
            time.sleep(0.2)
        assert (tmp_path / "progress" / "group0.rank0").is_file()
        trainers = _descendants(runner._groups[0].proc.pid, max_depth=1)
        assert trainers
        for pid in trainers:
            os.kill(pid, signal.SIGSTOP)
        th.join(300)
        assert not th.is_alive() and result.get("rc") == 0, result
        assert "made no progress" in capfd.readouterr().out
        second = (logs / "group_0.1.log").read_text()
        assert "step 799] should_commit=True" in second
        assert "step 799] should_commit=True" not in first.read_text()
    finally:
        for gp in runner._groups:
            if gp.proc is not None:
                _kill_tree(gp.proc.pid)
