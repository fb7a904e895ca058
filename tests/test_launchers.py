"""Launch helpers on CPU: the Slurm runner/punisher against fake ``squeue``/``sbatch``/``scancel``
on PATH, the torchx component (skipped without torchx), the stand-alone lighthouse CLI, and the
stream helpers on a host without an accelerator."""
import os
import stat
import subprocess
import sys
import time
import urllib.request

import pytest
import torch
from conftest import free_port


def _fake_tool(dirpath, name, body):
    p = os.path.join(dirpath, name)
    with open(p, "w") as f:
        f.write("#!/bin/sh\n" + body + "\n")
    os.chmod(p, os.stat(p).st_mode | stat.S_IEXEC)


def test_slurm_runner_and_punisher_with_fake_tools(tmp_path, monkeypatch):
    from torchft_b200.launch import slurm

    jobs = tmp_path / "jobs"
    jobs.write_text("ft_0\nunrelated\n")
    log = tmp_path / "calls.log"
    _fake_tool(tmp_path, "squeue", f"cat {jobs}")
    _fake_tool(tmp_path, "sbatch", f'echo "sbatch $@" >> {log}; for a in "$@"; do case $a in --job-name=*) echo "${{a#--job-name=}}" >> {jobs};; esac; done')
    _fake_tool(tmp_path, "scancel", f'echo "scancel $@" >> {log}; n="${{1#--name=}}"; grep -v "^$n$" {jobs} > {jobs}.tmp; mv {jobs}.tmp {jobs}')
    monkeypatch.setenv("PATH", f"{tmp_path}:{os.environ['PATH']}")

    assert slurm._running() == {"ft_0"}
    # one pass of the runner: replica 1 is missing and gets submitted with its environment
    monkeypatch.setattr(slurm.time, "sleep", lambda s: (_ for _ in ()).throw(KeyboardInterrupt()))
    with pytest.raises(KeyboardInterrupt):
        slurm.runner(2, 1, 8, "http://lh:29510", ["train_hsdp.py", "--model", "llama3-8b"])
    calls = log.read_text()
    assert "--job-name=ft_1" in calls and "REPLICA_GROUP_ID=1 NUM_REPLICA_GROUPS=2 TORCHFT_LIGHTHOUSE=http://lh:29510" in calls
    assert "train_hsdp.py --model llama3-8b" in calls and "--job-name=ft_0" not in calls
    assert slurm._running() == {"ft_0", "ft_1"}
    slurm.kill_one()
    assert len(slurm._running()) == 1
    slurm.kill_all()
    assert slurm._running() == set()


def test_torchx_component_shape():
    pytest.importorskip("torchx")
    from torchft_b200.launch.torchx import hsdp

    app = hsdp("--steps", "5", replicas=3, workers_per_replica=2, script="train_ddp.py")
    assert [r.name for r in app.roles] == ["replica_0", "replica_1", "replica_2"]
    assert app.roles[1].env["REPLICA_GROUP_ID"] == "1" and app.roles[1].env["NUM_REPLICA_GROUPS"] == "3"
    assert "--master_port=29601" in app.roles[1].args and app.roles[1].args[-2:] == ["--steps", "5"]


def test_torchx_component_without_torchx_raises_clearly():
    try:
        import torchx  # noqa: F401
        pytest.skip("torchx is installed")
    except ImportError:
        pass
    from torchft_b200.launch.torchx import hsdp

    with pytest.raises(RuntimeError, match="torchx"):
        hsdp()


def test_lighthouse_cli_serves_quorum_and_dashboard():
    from datetime import timedelta

    from torchft_b200._ftcp import LighthouseClient

    import socket

    s = socket.socket(socket.AF_INET6)
    s.bind(("::", 0))
    port = s.getsockname()[1]
    s.close()
    proc = subprocess.Popen([sys.executable, "-m", "torchft_b200.lighthouse_cli", "--bind", f"[::]:{port}", "--min_replicas", "1",
                             "--join_timeout_ms", "100", "--quorum_tick_ms", "10"],
                            cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), stdout=subprocess.PIPE,
                            stderr=subprocess.PIPE)
    try:
        deadline, q = time.time() + 30, None
        while time.time() < deadline:
            try:
                q = LighthouseClient(f"http://127.0.0.1:{port}", timedelta(seconds=1)).quorum("cli", timedelta(seconds=5))
                break
            except Exception:
                time.sleep(0.2)
        assert q is not None and q.quorum_id == 1 and [p.replica_id for p in q.participants] == ["cli"]
        page = urllib.request.urlopen(f"http://127.0.0.1:{port}/status", timeout=5).read().decode()
        assert "cli" in page
    finally:
        proc.terminate()
        proc.wait(timeout=10)
    # a missing required flag is reported, not ignored
    r = subprocess.run([sys.executable, "-m", "torchft_b200.lighthouse_cli"], capture_output=True, text=True, timeout=60,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode != 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="CPU-only behaviour")
def test_stream_helpers_are_noops_without_an_accelerator():
    from torchft_b200.utils.streams import get_stream_context, record_event, synchronize

    with get_stream_context(None):
        pass
    assert record_event() is None
    synchronize()


def test_runner_restarts_a_group_after_an_injected_segfault(tmp_path):
    """Punisher.inject("segfault") sends SIGSEGV to a group's trainer processes (not to its launcher); the launcher
    reports the failure by exiting non-zero and the runner starts the group again."""
    import threading
    import time
    from pathlib import Path

    from torchft_b200.launch.runner import Punisher, Runner, _descendants

    repo = Path(__file__).resolve().parent.parent
    pid_file = str(tmp_path / "pids.json")
    runner = Runner([str(repo / "tests" / "_sleepy_worker.py")], num_groups=1, base_port=free_port(8),
                    max_restarts=2, pid_file=pid_file, poll_secs=0.2, log_dir=str(tmp_path / "logs"),
                    extra_env={"SLEEPY_DIR": str(tmp_path)})
    result = {}
    th = threading.Thread(target=lambda: result.setdefault("rc", runner.run()), daemon=True)
    th.start()
    try:
        log0 = tmp_path / "logs" / "group_0.0.log"
        end = time.monotonic() + 120
        while not (log0.exists() and "incarnation 1" in log0.read_text()):
            assert time.monotonic() < end and th.is_alive()
            time.sleep(0.2)
        assert Punisher(pid_file).inject("segfault", group=0) == 0
        th.join(180)
        assert not th.is_alive() and result.get("rc") == 0, result
        assert "incarnation 2" in (tmp_path / "logs" / "group_0.1.log").read_text()
    finally:
        for gp in runner._groups:
            if gp.proc is not None and gp.proc.poll() is None:
                for q in _descendants(gp.proc.pid) + [gp.proc.pid]:
                    try:
                        os.kill(q, 9)
                    except ProcessLookupError:
                        pass


def test_punisher_hang_stops_then_kills_the_group(tmp_path):
    """Punisher.inject("hang"): the trainers are stopped (alive but silent) and, after ``hang_secs``, the whole group is
    killed so that the runner replaces it."""
    import threading
    import time
    from pathlib import Path

    from torchft_b200.launch.runner import Punisher, Runner, _descendants

    repo = Path(__file__).resolve().parent.parent
    pid_file = str(tmp_path / "pids.json")
    runner = Runner([str(repo / "tests" / "_sleepy_worker.py")], num_groups=1, base_port=free_port(8),
                    max_restarts=2, pid_file=pid_file, poll_secs=0.2, log_dir=str(tmp_path / "logs"),
                    extra_env={"SLEEPY_DIR": str(tmp_path)})
    result = {}
    th = threading.Thread(target=lambda: result.setdefault("rc", runner.run()), daemon=True)
    th.start()
    try:
        log0 = tmp_path / "logs" / "group_0.0.log"
        end = time.monotonic() + 120
        while not (log0.exists() and "incarnation 1" in log0.read_text()):
            assert time.monotonic() < end and th.is_alive()
            time.sleep(0.2)
        trainer = _descendants(runner._groups[0].proc.pid, max_depth=1)[0]
        stopper = threading.Thread(target=lambda: Punisher(pid_file).inject("hang", group=0, hang_secs=2.0), daemon=True)
        stopper.start()
        end = time.monotonic() + 10
        state = ""
        while time.monotonic() < end and state != "T":
            try:
                state = open(f"/proc/{trainer}/stat").read().rsplit(")", 1)[1].split()[0]
            except OSError:
                break
            time.sleep(0.05)
        assert state == "T"  # stopped, not dead
        stopper.join(30)
        th.join(180)
        assert not th.is_alive() and result.get("rc") == 0, result
        assert "incarnation 2" in (tmp_path / "logs" / "group_0.1.log").read_text()
    finally:
        for gp in runner._groups:
            if gp.proc is not None and gp.proc.poll() is None:
                for q in _descendants(gp.proc.pid) + [gp.proc.pid]:
                    try:
                        os.kill(q, 9)
                    except ProcessLookupError:
                        pass
