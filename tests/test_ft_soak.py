"""Soak: many injected replica failures in a row (alternating between the two replica groups), each
followed by a restart and a live heal from the surviving group.  Pass criteria: every failure was
injected, nothing hung (the run is bounded), both groups end on the same step with identical weights.
The baseline's acceptance bar for recovery is "zero hangs across 100 injected failures"; the number
here is FTB200_SOAK_FAILURES (default 100, under a minute)."""
import os
import threading
import time
from typing import List, Optional, Tuple

from ft_harness import EventInjector, InjectedFailure, Runner, run_replicas
from test_manager_integ import _assert_same, ddp_train_loop
from torchft_b200._ftcp import LighthouseServer


class SoakInjector(EventInjector):
    """Fails the planned (replica, step) pairs one at a time; while a failed group is restarting, the
    survivor is held (bounded) so that it neither finishes nor runs far ahead before the heal."""

    def __init__(self, plan: List[Tuple[int, int]]) -> None:
        super().__init__()
        self._plan = list(plan)
        self._restarting: Optional[int] = None
        self._cv = threading.Condition()

    def notify_restarted(self) -> None:
        with self._cv:
            self._restarting = None
            self._cv.notify_all()

    def check(self, replica, rank, step, pg=None) -> None:
        with self._cv:
            if self._restarting is not None and self._restarting != replica:
                self._cv.wait_for(lambda: self._restarting is None, timeout=5.0)
            if self._restarting is None and self._plan and self._plan[0][0] == replica and step >= self._plan[0][1]:
                self._plan.pop(0)
                self._restarting = replica
                self.count += 1
                raise InjectedFailure(f"soak failure #{self.count}: replica={replica} step={step}")

    @property
    def remaining(self) -> int:
        return len(self._plan)


def test_many_failures_in_a_row_no_hang():
    n = int(os.environ.get("FTB200_SOAK_FAILURES", "100"))
    plan = [(i % 2, 3 * i + 2) for i in range(n)]
    total_steps = 3 * n + 6
    lh = LighthouseServer("[::]:0", 1, join_timeout_ms=100, quorum_tick_ms=10, heartbeat_timeout_ms=500)
    try:
        inj = SoakInjector(plan)
        runners = [Runner(i, lh.address(), inj, None, attempts=n + 2) for i in range(2)]  # type: ignore[arg-type]
        for r in runners:
            r.train_loop = lambda rank, store_port, runner: ddp_train_loop(rank, store_port, runner, total_steps=total_steps,
                                                                          batch=8, use_async_quorum=False)
        t0 = time.time()
        res = run_replicas(runners, timeout=60 + 6 * n)
        elapsed = time.time() - t0
        assert inj.count == n and inj.remaining == 0
        assert all(r[0]["step"] == total_steps for r in res)
        _assert_same(res)
        print(f"soak: {n} failures healed in {elapsed:.1f} s")
    finally:
        lh.shutdown()
