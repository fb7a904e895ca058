import threading
import time
from datetime import timedelta
from unittest.mock import patch

import pytest
from torch.futures import Future

from torchft_b200 import futures as F
from torchft_b200.checkpointing._rwlock import RWLock


def test_future_wait_and_timeout():
    fut = Future()
    with pytest.raises(TimeoutError):
        F.future_wait(fut, timedelta(seconds=0.05))
    fut.set_result(7)
    assert F.future_wait(fut, timedelta(seconds=1)) == 7
    bad = Future()
    bad.set_exception(RuntimeError("boom"))
    with pytest.raises(RuntimeError, match="boom"):
        F.future_wait(bad, timedelta(seconds=1))


def test_future_timeout_fires_and_passes_through():
    slow = Future()
    timed = F.future_timeout(slow, timedelta(seconds=0.05))
    with pytest.raises(TimeoutError):
        timed.wait()
    ok = Future()
    timed2 = F.future_timeout(ok, timedelta(seconds=5))
    ok.set_result("v")
    assert timed2.wait() == "v"
    err = Future()
    timed3 = F.future_timeout(err, timedelta(seconds=5))
    err.set_exception(ValueError("x"))
    with pytest.raises(ValueError):
        timed3.wait()


def test_context_timeout():
    fired = threading.Event()
    with F.context_timeout(fired.set, timedelta(seconds=5)):
        pass
    time.sleep(0.05)
    assert not fired.is_set()
    with F.context_timeout(fired.set, timedelta(seconds=0.02)):
        time.sleep(0.2)
    assert fired.is_set()


def test_watchdog_exits_when_callback_is_stuck():
    mgr = F._TimeoutManager()
    mgr._watchdog_interval = timedelta(seconds=0.1)
    exited = threading.Event()
    release = threading.Event()
    with patch.object(F._TimeoutManager, "_exit", staticmethod(exited.set)):
        mgr.call_later(timedelta(seconds=0.01), lambda: release.wait(5))
        assert exited.wait(3)
    release.set()
    mgr.shutdown()


def test_rwlock_readers_writer():
    lock = RWLock(timeout=0.2)
    lock.r_acquire()
    lock.r_acquire()  # many readers
    with pytest.raises(TimeoutError):
        lock.w_acquire()
    lock.r_release()
    lock.r_release()
    with lock.w_lock():
        assert lock.w_locked()
        with pytest.raises(TimeoutError):
            lock.r_acquire()
    with lock.r_lock():
        pass


def test_rwlock_writer_preference():
    lock = RWLock(timeout=2)
    lock.r_acquire()
    got = []
    t = threading.Thread(target=lambda: (lock.w_acquire(), got.append("w"), lock.w_release()))
    t.start()
    time.sleep(0.05)
    fast = RWLock.__dict__  # noqa: F841
    lock2_err = []

    def late_reader():
        try:
            lock.r_acquire()
            got.append("r")
            lock.r_release()
        except TimeoutError as e:
            lock2_err.append(e)

    r = threading.Thread(target=late_reader)
    r.start()
    time.sleep(0.05)
    assert got == []  # the late reader queues behind the waiting writer
    lock.r_release()
    t.join()
    r.join()
    assert got == ["w", "r"]


def test_stream_timeout_logic_with_a_fake_event(monkeypatch):
    """stream_timeout: the callback runs only when the recorded event has not completed by the deadline, and the event
    is handed to the deletion queue instead of being destroyed on the timer thread (torchft/futures_test.py
    test_stream_timeout; the CUDA event is faked so that the logic runs on CPU)."""
    import threading
    import time
    from datetime import timedelta

    import torch

    from torchft_b200 import futures as F

    class FakeEvent:
        done = False
        recorded = 0

        def record(self):
            FakeEvent.recorded += 1

        def query(self):
            return FakeEvent.done

    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "Event", FakeEvent)
    fired = threading.Event()
    FakeEvent.done = False
    F.stream_timeout(fired.set, timedelta(milliseconds=30))
    assert fired.wait(5) and FakeEvent.recorded == 1
    fired.clear()
    FakeEvent.done = True  # the stream finished in time
    F.stream_timeout(fired.set, timedelta(milliseconds=30))
    time.sleep(0.3)
    assert not fired.is_set() and FakeEvent.recorded == 2
    assert F._TIMEOUT_MANAGER._drain_del_queue() >= 1  # parked events are released by a later caller


def test_timer_wakes_for_earlier_deadlines_and_sweeps_cancelled_timers():
    """A timer armed after a later one still fires on time (the timer thread is woken because the new deadline is the
    earliest), and cancelled timers do not pile up in the heap."""
    import threading
    import time
    from datetime import timedelta

    from torchft_b200 import futures as F

    tm = F._TIMEOUT_MANAGER
    late, early = threading.Event(), threading.Event()
    h_late = tm.call_later(timedelta(seconds=30), late.set)
    t0 = time.monotonic()
    tm.call_later(timedelta(milliseconds=50), early.set)
    assert early.wait(2) and time.monotonic() - t0 < 1.0
    assert not late.is_set()
    h_late.cancel()
    handles = [tm.call_later(timedelta(seconds=60), lambda: None) for _ in range(F._COMPACT_ABOVE + 200)]
    for h in handles:
        h.cancel()
    tm.call_later(timedelta(seconds=60), lambda: None).cancel()  # this push sweeps the cancelled ones
    assert len(tm._heap) < 300
