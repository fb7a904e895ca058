"""The allocation-aware orchestrator (torchft_b200/launch/orchestrator.py) with stand-in trainers: retry on the same
allocation, a new allocation after repeated failures, giving a group up, and failure injection into a running group."""
import os
import sys
import time

from torchft_b200.launch.orchestrator import (Allocation, FailureController, GpuPoolAllocator, Orchestrator,
                                              SlurmAllocator)


def _script(tmp_path, body: str) -> str:
    p = tmp_path / "trainer.py"
    p.write_text(body)
    return str(p)


def test_gpu_pool_prefers_slices_that_have_not_failed():
    pool = GpuPoolAllocator([0, 1, 2, 3, 4, 5], 2)
    a, b = pool.acquire(0), pool.acquire(1)
    assert a.env["CUDA_VISIBLE_DEVICES"] == "0,1" and b.env["CUDA_VISIBLE_DEVICES"] == "2,3"
    pool.release(a, failed=True)          # GPUs 0,1 look broken
    c = pool.acquire(0)
    assert c.env["CUDA_VISIBLE_DEVICES"] == "4,5"   # the spare slice first
    pool.release(c, failed=True)
    d = pool.acquire(0)
    assert d.env["CUDA_VISIBLE_DEVICES"] == "0,1"   # no clean slice left: the oldest suspect comes back


def test_retries_then_moves_to_a_new_allocation_and_finishes(tmp_path):
    # the trainer fails while it sees GPU 0 (a "broken" device) and succeeds elsewhere
    script = _script(tmp_path, "import os, sys\nsys.exit(3 if '0' in os.environ['CUDA_VISIBLE_DEVICES'].split(',') else 0)\n")
    orch = Orchestrator(2, GpuPoolAllocator([0, 1, 2], 1), lambda g, alloc: [sys.executable, script],
                        lighthouse_addr="http://127.0.0.1:1", proc_attempts=2, max_attempts=8, retry_delay_s=0.01,
                        log_dir=str(tmp_path / "logs"))
    groups = orch.run()
    assert all(g.done and not g.abandoned for g in groups.values())
    g0 = groups[0]
    assert g0.attempts == 3 and g0.allocations == ["gpus-0", "gpus-2"]   # two failures on GPU 0, then the spare
    assert groups[1].attempts == 1
    assert sorted(os.listdir(tmp_path / "logs")) == ["group0.attempt1.log", "group0.attempt2.log", "group0.attempt3.log",
                                                    "group1.attempt1.log"]


def test_gives_a_group_up_after_max_attempts(tmp_path):
    script = _script(tmp_path, "import os, sys\nsys.exit(0 if os.environ['REPLICA_GROUP_ID'] == '1' else 5)\n")
    orch = Orchestrator(2, GpuPoolAllocator([0, 1], 1), lambda g, alloc: [sys.executable, script],
                        lighthouse_addr="http://127.0.0.1:1", proc_attempts=2, max_attempts=5, retry_delay_s=0.01)
    groups = orch.run()
    assert groups[0].abandoned and groups[0].attempts == 5 and not groups[0].done
    assert groups[1].done


def test_failure_controller_kills_a_running_group_which_is_then_restarted(tmp_path):
    marker = tmp_path / "runs"
    script = _script(tmp_path, f"import os, time\nopen(r'{marker}', 'a').write('x')\n"
                               f"time.sleep(0.2 if len(open(r'{marker}').read()) > 1 else 30)\n")
    orch = Orchestrator(1, GpuPoolAllocator([0], 1), lambda g, alloc: [sys.executable, script],
                        lighthouse_addr="http://127.0.0.1:1", retry_delay_s=0.01)
    failures = FailureController(orch.groups, mtbf_secs=0.3, kinds=["kill"], seed=1)
    t0 = time.time()
    groups = orch.run(failures)
    assert groups[0].done and groups[0].attempts >= 2 and time.time() - t0 < 25
    assert failures.injected and failures.injected[0][2] == "kill"


def test_slurm_allocator_builds_the_commands():
    calls = []

    class R:
        stdout, stderr = "", "salloc: Granted job allocation 4242\n"

    def run(cmd, **kw):
        calls.append(cmd)
        return R()

    alloc = SlurmAllocator(nodes=2, salloc_args=["--partition=gpu"], run=run)
    a = alloc.acquire(3)
    assert isinstance(a, Allocation) and a.prefix == ["srun", "--jobid=4242"] and a.env["SLURM_JOB_ID"] == "4242"
    assert calls[0][:4] == ["salloc", "--no-shell", "--nodes=2", "--job-name=ft_3"]
    alloc.release(a, failed=True)
    assert calls[1] == ["scancel", "4242"]
