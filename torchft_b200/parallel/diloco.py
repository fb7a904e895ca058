"""Streaming DiLoCo on the explicit Llama engine.

Every replica group trains on its own with :class:`~torchft_b200.parallel.hsdp.ShardedLlamaTrainer`
(no per-step replica allreduce); every ``sync_every / n_fragments`` inner steps one fragment
of the model -- a contiguous run of the trainer's flat units -- exchanges its
pseudo-gradient ``last global weights - local weights`` with the other groups and takes an
outer Nesterov step.  The schedule, the commit rule and the state-dict keys are those of
:class:`torchft_b200.local_sgd.DiLoCo` (torchft/local_sgd.py:176-796); what differs is the
data layout: weights, backup, pseudo-gradient and outer momentum are the trainer's flat
fp32 shards, so one fragment synchronisation is, per unit,

* one fused kernel for ``average_over_groups(fp8(backup - master))``
  (:meth:`torchft_b200.manager.Manager.allreduce_delta`), and
* one fused kernel for momentum, Nesterov step, new backup and blend with the local
  weights (:func:`torchft_b200.ops.diloco.outer_step_`),

followed by the cast of the new master weights to the bf16 compute copy.  With sharding
inside the group every rank exchanges its own shard with the same-numbered rank of the
other groups, so the exchanged bytes per GPU fall with the group size.
"""

from __future__ import annotations

import logging
from contextlib import nullcontext
from typing import Dict, List, Optional

import torch
from torch.distributed.distributed_c10d import Work

from ..manager import Manager
from ..ops.diloco import outer_step_
from .hsdp import ShardedLlamaTrainer

logger = logging.getLogger(__name__)


def split_units(numels: List[int], n_fragments: int) -> List[List[int]]:
    """Contiguous groups of unit indices with roughly equal element counts; every fragment
    gets at least one unit."""
    U = len(numels)
    if not 1 <= n_fragments <= U:
        raise ValueError(f"need 1 <= n_fragments <= {U} units, got {n_fragments}")
    total, out, cur, acc = float(sum(numels)), [], [], 0.0
    for u, n in enumerate(numels):
        cur.append(u)
        acc += n
        left_units, left_frags = U - u - 1, n_fragments - len(out) - 1
        if left_frags > 0 and (acc >= total * (len(out) + 1) / n_fragments or left_units == left_frags):
            out.append(cur)
            cur = []
    out.append(cur)
    assert len(out) == n_fragments and all(out), out
    return out


class _EngineFragment:
    def __init__(self, owner: "EngineDiLoCo", fragment_id: int, units: List[int]) -> None:
        t = owner.trainer
        self.owner, self.id, self.units = owner, fragment_id, units
        self.backup = [t.master[u].clone() for u in units]
        self.grad = [torch.empty_like(t.master[u]) for u in units]
        self.momentum = [torch.zeros_like(t.master[u]) for u in units]
        self.outer_steps = 0
        self.works: List[Work] = []
        self.event: Optional[torch.cuda.Event] = None

    # ---- healing state
    def register(self, manager: Manager) -> None:
        def save() -> Dict[str, object]:
            return {
                "original_parameters": {f"unit{u}": b.clone() for u, b in zip(self.units, self.backup)},
                "outer_momentum": {f"unit{u}": m.clone() for u, m in zip(self.units, self.momentum)},
                "outer_steps": self.outer_steps,
            }

        def load(sd: Dict[str, object]) -> None:
            for u, b, m in zip(self.units, self.backup, self.momentum):
                b.copy_(sd["original_parameters"][f"unit{u}"])  # type: ignore[index]
                m.copy_(sd["outer_momentum"][f"unit{u}"])  # type: ignore[index]
            self.outer_steps = int(sd["outer_steps"])  # type: ignore[arg-type]

        manager.register_state_dict_fn(f"StreamingDiLoCoFragment_{self.id}", load, save)

    # ---- synchronisation
    def prepare(self) -> None:
        o, t = self.owner, self.owner.trainer
        assert not self.works
        early = o.fragment_sync_delay > 0
        if early:  # inner steps continue during the exchange: take the difference now
            for b, g, u in zip(self.backup, self.grad, self.units):
                torch.sub(b, t.master[u], out=g)
        stream = o.stream
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream) if stream is not None else nullcontext():
            if o.record_timing:
                ev0 = torch.cuda.Event(enable_timing=True)
                ev0.record()
            for b, g, u in zip(self.backup, self.grad, self.units):
                if early:
                    self.works.append(o.manager.allreduce(g, should_quantize=o.should_quantize))
                else:
                    self.works.append(o.manager.allreduce_delta(g, b, t.master[u], should_quantize=o.should_quantize))
            if o.record_timing:
                ev1 = torch.cuda.Event(enable_timing=True)
                ev1.record()
                o.exchange_timings.append((ev0, ev1))

    def perform(self) -> bool:
        o, t = self.owner, self.owner.trainer
        assert self.works
        stream = o.stream
        with torch.cuda.stream(stream) if stream is not None else nullcontext():
            for w in self.works:
                w.wait()
        if stream is not None:
            torch.cuda.current_stream().wait_stream(stream)
        self.works = []
        committed = o.manager.should_commit()
        for b, g, m, u in zip(self.backup, self.grad, self.momentum, self.units):
            if committed:
                outer_step_(g, m, b, t.master[u], lr=o.outer_lr, momentum_coef=o.outer_momentum,
                            alpha=o.fragment_update_alpha, nesterov=o.nesterov, first_step=self.outer_steps == 0)
            else:
                t.master[u].copy_(b)
            t.p_shard[u].copy_(t.master[u])
        if committed:
            self.outer_steps += 1
        t.invalidate_gathered(self.units)
        return committed


class EngineDiLoCo:
    """Drives a :class:`ShardedLlamaTrainer` (constructed with ``manager=None``) under
    (streaming) DiLoCo.  ``train_step`` is one inner step plus whatever fragment work falls
    on it.  The manager must use a synchronous quorum; register the trainer's own
    ``state_dict``/``load_state_dict`` with the manager as well so that a healing replica
    receives the live weights and inner optimizer state."""

    def __init__(self, trainer: ShardedLlamaTrainer, manager: Manager, n_fragments: int = 1, sync_every: int = 100,
                 outer_lr: float = 0.7, outer_momentum: float = 0.9, nesterov: bool = True, should_quantize: bool = False,
                 fragment_sync_delay: int = 0, fragment_update_alpha: float = 0.0, record_timing: bool = False) -> None:
        if trainer.manager is not None:
            raise ValueError("the trainer must not allreduce gradients per step (construct it with manager=None)")
        if manager._use_async_quorum:
            raise ValueError("DiLoCo requires a manager with use_async_quorum=False")
        if sync_every < n_fragments or sync_every % n_fragments:
            raise ValueError("sync_every must be a positive multiple of the number of fragments")
        self._every = sync_every // n_fragments
        if not 0 <= fragment_sync_delay < self._every:
            raise ValueError("fragment_sync_delay must be shorter than the interval between fragment syncs")
        if not 0.0 <= fragment_update_alpha <= 1.0:
            raise ValueError("fragment_update_alpha must be between 0 and 1")
        self.trainer, self.manager = trainer, manager
        self.outer_lr, self.outer_momentum, self.nesterov = outer_lr, outer_momentum, nesterov
        self.should_quantize = should_quantize
        self.fragment_sync_delay, self.fragment_update_alpha = fragment_sync_delay, fragment_update_alpha
        self.stream = torch.cuda.Stream(trainer.device) if trainer.device.type == "cuda" else None
        self.fragments = [_EngineFragment(self, i, units)
                          for i, units in enumerate(split_units(trainer.shard_numel, n_fragments))]
        for f in self.fragments:
            f.register(manager)
        self._local_step = 0
        self.last_sync_committed: Optional[bool] = None
        self.commits = 0
        # with record_timing on CUDA: per synchronisation the (start, end) event pairs of its
        # parts on the training stream, and per exchange the pair on the communication stream
        self.record_timing = record_timing and self.stream is not None
        self.timings: List[List[tuple]] = []
        self.exchange_timings: List[tuple] = []
        # with record_timing: host time (monotonic seconds) at which this group's training stream reached each
        # synchronisation; comparing them across the groups of one host gives their drift
        self.arrivals: List[float] = []
        self._arrival_threads: List = []

    def _stamp_arrival(self) -> None:
        """Host time at which the training stream reaches this point, taken by a helper thread that waits for an
        event: the training thread itself must not wait for the device here, or it would lose the lead over the
        device that hides the wait for slower groups."""
        import threading
        import time

        ev = torch.cuda.Event()
        ev.record()
        slot = len(self.arrivals)
        self.arrivals.append(float("nan"))

        def wait() -> None:
            ev.synchronize()
            self.arrivals[slot] = time.monotonic()

        t = threading.Thread(target=wait, name="diloco_arrival", daemon=True)
        t.start()
        self._arrival_threads.append(t)

    def arrival_times(self) -> List[float]:
        """The recorded arrivals, once the device has passed all of them."""
        for t in self._arrival_threads:
            t.join()
        self._arrival_threads.clear()
        return list(self.arrivals)

    def _timed(self, fn, new_sync: bool):
        if not self.record_timing:
            return fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn()
        b.record()
        if new_sync:
            self.timings.append([])
        self.timings[-1].append((a, b))
        return out

    def _current(self) -> _EngineFragment:
        return self.fragments[self.manager.current_step() % len(self.fragments)]

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.manager.disallow_state_dict_read()
        loss = self.trainer.train_step(tokens, targets)
        self.manager.allow_state_dict_read()
        self._local_step += 1
        if self._local_step == self._every - self.fragment_sync_delay:
            if self.record_timing:
                self._stamp_arrival()

            def begin() -> None:
                self.manager.start_quorum()  # synchronous: a replica that is behind heals here
                self._current().prepare()

            self._timed(begin, new_sync=True)
        if self._local_step == self._every:
            self.last_sync_committed = self._timed(lambda: self._current().perform(), new_sync=False)
            self.commits += int(bool(self.last_sync_committed))
            self._local_step = 0
        return loss
