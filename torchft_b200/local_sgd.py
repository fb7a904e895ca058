"""Communication-sparse training: LocalSGD, DiLoCo and streaming DiLoCo.

All three run the inner optimizer locally and synchronise through the manager only every
``sync_every`` inner steps, so a replica failure costs at most one synchronisation window:

* :class:`LocalSGD` averages the *parameters* (https://arxiv.org/abs/1805.09767);
* :class:`DiLoCo` averages *pseudo-gradients* (last synchronised weights minus current
  weights) and applies them with an outer optimizer, typically Nesterov SGD
  (https://arxiv.org/abs/2311.08105);
* with several model fragments :class:`DiLoCo` is streaming DiLoCo
  (https://arxiv.org/abs/2501.18512): fragments take turns, the allreduce of a fragment
  is started ``fragment_sync_delay`` inner steps before it is needed, and the new global
  weights are blended with the local ones by ``fragment_update_alpha``.

Semantics (hook points, scheduling, state-dict keys, argument validation) follow
torchft/local_sgd.py:46-796; pseudo-gradient formation, bucket packing and the outer
update run as fused multi-tensor kernels on CUDA (see :mod:`torchft_b200.ops.diloco`).
"""

from __future__ import annotations

import logging
import math
import os
from contextlib import nullcontext
from types import TracebackType
from typing import Any, Dict, List, Optional, Tuple, Type, Union

import torch
from torch import nn, optim
from torch.distributed.distributed_c10d import Work
from torch.utils.hooks import RemovableHandle

from .manager import Manager

try:
    from torch.distributed.tensor import DTensor
except Exception:  # pragma: no cover
    DTensor = None  # type: ignore

logger = logging.getLogger(__name__)

USE_BUCKETIZATION_ENV: str = "TORCHFT_USE_BUCKETIZATION"


def extract_local_tensor(t: torch.Tensor) -> torch.Tensor:
    """A detached *copy* of the local shard of ``t`` (``t`` itself for plain tensors)."""
    if DTensor is not None and isinstance(t, DTensor):
        return t.to_local().clone()
    return t.clone()


def _local_view(t: torch.Tensor) -> torch.Tensor:
    if DTensor is not None and isinstance(t, DTensor):
        return t.to_local()
    return t


def _assign(p: torch.Tensor, value: torch.Tensor, non_blocking: bool = False) -> None:
    """``p.data <- value`` where ``value`` is the local shard when ``p`` is a DTensor."""
    _local_view(p.data).copy_(value, non_blocking=non_blocking)


class LocalSGD:
    """Context manager: every ``sync_every`` optimizer steps the parameters are averaged
    across replicas (quorum -> allreduce -> commit vote -> copy back).  If the window
    fails to commit, local weights are kept and the next window tries again.

    ``bucket_cap_mb``: when given, the parameter copies of one dtype and device are packed into flat buffers of at most
    that size and each buffer is one allreduce (a model with hundreds of small parameters then costs a handful of
    collectives instead of hundreds); ``None`` keeps one allreduce per parameter, as the reference does
    (torchft/local_sgd.py:160-173).  The averaged values are the same either way."""

    def __init__(self, manager: Manager, model: nn.Module, optimizer: optim.Optimizer, sync_every: int,
                 bucket_cap_mb: Optional[int] = None) -> None:
        assert sync_every >= 1, "sync_every must be greater than or equal to 1"
        assert bucket_cap_mb is None or bucket_cap_mb > 0, "bucket_cap_mb must be positive"
        self._manager, self._model, self._local_optimizer = manager, model, optimizer
        self._sync_every = sync_every
        self._bucket_cap_bytes = None if bucket_cap_mb is None else bucket_cap_mb * 1024 * 1024
        self._local_step = 0
        self._hooks: List[RemovableHandle] = []

    def __enter__(self) -> "LocalSGD":
        self._hooks.append(self._local_optimizer.register_step_pre_hook(self._step_pre_hook))
        self._hooks.append(self._local_optimizer.register_step_post_hook(self._step_post_hook))
        return self

    def __exit__(self, exc_type: Optional[Type[BaseException]], exc_value: Optional[BaseException],
                 tb: Optional[TracebackType]) -> bool:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        return False

    def _step_pre_hook(self, _o: optim.Optimizer, _a: Tuple[Any, ...], _k: Dict[str, Any]) -> None:
        # peers must not read weights that are half way through an optimizer step
        self._manager.disallow_state_dict_read()

    def _step_post_hook(self, _o: optim.Optimizer, _a: Tuple[Any, ...], _k: Dict[str, Any]) -> None:
        self._manager.allow_state_dict_read()
        self._local_step += 1
        if self._local_step >= self._sync_every:
            self.sync()

    def sync(self) -> None:
        """Average the weights across the replicas now."""
        self._manager.start_quorum()
        self._perform_sync()
        self._local_step = 0

    def _perform_sync(self) -> None:
        averaged = self._average()
        if self._manager.should_commit():
            with torch.no_grad():
                for p, avg in zip(self._model.parameters(), averaged):
                    _assign(p, avg)

    def _average(self) -> List[torch.Tensor]:
        if self._bucket_cap_bytes is not None:
            return self._average_bucketed(self._bucket_cap_bytes)
        copies = [extract_local_tensor(p.data) for p in self._model.parameters()]
        works = [self._manager.allreduce(c) for c in copies]
        for w in works:
            w.wait()
        return copies

    def _average_bucketed(self, cap_bytes: int) -> List[torch.Tensor]:
        """Pack the local values into flat buffers per (dtype, device), allreduce each buffer once and return views
        into the buffers in parameter order.  A parameter larger than the cap gets a buffer of its own."""
        locals_ = [_local_view(p.data) for p in self._model.parameters()]
        out: List[Optional[torch.Tensor]] = [None] * len(locals_)
        groups: Dict[Tuple[torch.dtype, torch.device], List[int]] = {}
        for i, t in enumerate(locals_):
            groups.setdefault((t.dtype, t.device), []).append(i)
        works = []
        for (dtype, device), idxs in groups.items():
            start = 0
            while start < len(idxs):
                end, nbytes = start, 0
                while end < len(idxs) and (end == start or nbytes + locals_[idxs[end]].numel() * locals_[idxs[end]].element_size() <= cap_bytes):
                    nbytes += locals_[idxs[end]].numel() * locals_[idxs[end]].element_size()
                    end += 1
                flat = torch.empty(sum(locals_[i].numel() for i in idxs[start:end]), dtype=dtype, device=device)
                off = 0
                for i in idxs[start:end]:
                    n = locals_[i].numel()
                    view = flat[off:off + n].view(locals_[i].shape)
                    view.copy_(locals_[i])
                    out[i] = view
                    off += n
                works.append(self._manager.allreduce(flat))
                start = end
        for w in works:
            w.wait()
        return out  # type: ignore[return-value]


class _StreamingDiLoCoFragment:
    """One fragment of the model with its own backup of the last global weights, outer
    optimizer and communication stream."""

    bucket_cap_mb: int = 1 * 1024 * 1024 * 1024  # bytes, despite the historical name
    use_bucketization: bool = False

    def __init__(
        self,
        manager: Manager,
        model_fragment: nn.Module,
        fragment_id: int,
        fragment_sync_offset: int,
        inner_optimizer: optim.Optimizer,
        outer_optimizer: optim.Optimizer,
        sync_every: int,
        backup_device: Optional[torch.device] = None,
        pin_memory: bool = True,
        use_bucketization: bool = False,
        bucket_cap_mb: Optional[int] = None,
        should_quantize: bool = False,
        fragment_sync_delay: int = 0,
        fragment_update_alpha: float = 0.0,
    ) -> None:
        if fragment_sync_offset > sync_every:
            raise ValueError("Fragment must be synced once before `sync_every` steps")
        assert sync_every >= 1, "sync_every must be greater than or equal to 1"
        self._fragment_id = fragment_id
        self._manager = manager
        self._model_fragment = model_fragment
        self._fragment_sync_offset = fragment_sync_offset
        self._local_optimizer = inner_optimizer
        self._outer_optimizer = outer_optimizer
        self._sync_every = sync_every
        self._backup_device = backup_device
        self._pin_memory = pin_memory
        self._fragment_sync_delay = fragment_sync_delay
        self._fragment_update_alpha = fragment_update_alpha
        self.should_quantize = should_quantize
        self._allreduce_work: List[Work] = []
        self._stream: Optional[torch.cuda.Stream] = torch.cuda.Stream() if torch.cuda.is_available() else None
        self._stop_event: Optional[torch.cuda.Event] = None
        if bucket_cap_mb is not None:
            self.bucket_cap_mb = int(bucket_cap_mb * 1024 * 1024)
        self.use_bucketization = os.getenv(USE_BUCKETIZATION_ENV, "False") == "True" or use_bucketization

        self._grads: Dict[str, torch.Tensor] = {}
        self._local_parameters: Dict[str, torch.Tensor] = {}
        self.original_parameters: Dict[str, torch.Tensor] = {}
        dev = self._backup_device or torch.device("cpu")
        for name, p in self._model_fragment.named_parameters():
            local = _local_view(p.data)
            t = torch.empty(*tuple(local.shape), dtype=local.dtype, device=dev)
            if self._pin_memory and t.device.type == "cpu" and torch.cuda.is_available():
                t = t.pin_memory()
            self.original_parameters[name] = t

    # ---- healing state ------------------------------------------------------------------
    def register_state_dict_fn(self) -> None:
        """Adds ``StreamingDiLoCoFragment_<id>`` -> ``{outer_optimizer, original_parameters}``
        to what the manager transfers when a replica heals."""
        key = f"StreamingDiLoCoFragment_{self._fragment_id}"

        def load_fn(sd: Dict[str, Dict[str, torch.Tensor]]) -> None:
            for name, value in sd["original_parameters"].items():
                if name in self.original_parameters:
                    self.original_parameters[name].copy_(value)
            self._outer_optimizer.load_state_dict(sd["outer_optimizer"])

        def save_fn() -> Dict[str, Dict[str, torch.Tensor]]:
            return {
                "outer_optimizer": self._outer_optimizer.state_dict(),
                "original_parameters": {n: t.clone() for n, t in self.original_parameters.items()},
            }

        self._manager.register_state_dict_fn(key, load_fn, save_fn)

    # ---- parameter bookkeeping ------------------------------------------------------------
    def save_parameters(self) -> None:
        """backup <- current model weights (the new global weights)."""
        with torch.profiler.record_function("torchft::local_sgd::save_parameters"), torch.no_grad():
            for name, p in self._model_fragment.named_parameters():
                self.original_parameters[name].copy_(_local_view(p.data), non_blocking=True)

    def _save_local_parameters(self) -> None:
        with torch.no_grad():
            for name, p in self._model_fragment.named_parameters():
                self._local_parameters[name] = extract_local_tensor(p.data)

    def restore_parameters(self) -> None:
        """model weights <- backup (the last global weights)."""
        with torch.profiler.record_function("torchft::local_sgd::restore_parameters"), torch.no_grad():
            for name, p in self._model_fragment.named_parameters():
                _assign(p, self.original_parameters[name], non_blocking=False)

    def _save_grads(self) -> None:
        """pseudo-gradient = last global weights - current local weights."""
        with torch.no_grad():
            for name, p in self._model_fragment.named_parameters():
                local = _local_view(p.data)
                self._grads[name] = self.original_parameters[name].to(local.device) - local

    def _set_grads(self) -> None:
        with torch.no_grad():
            for name, p in self._model_fragment.named_parameters():
                g = self._grads.pop(name)
                if DTensor is not None and isinstance(p, DTensor):
                    p.grad = DTensor.from_local(g, p.device_mesh, p.placements, shape=p.shape, stride=p.stride())
                else:
                    p.grad = g

    def _clear_local_parameters(self) -> None:
        self._local_parameters = {}

    def _merge_parameters(self) -> None:
        """weights <- lerp(new global, local, alpha): alpha 0 keeps the global weights."""
        with torch.no_grad():
            for name, p in self._model_fragment.named_parameters():
                _local_view(p.data).lerp_(self._local_parameters[name], self._fragment_update_alpha)

    # ---- synchronisation --------------------------------------------------------------------
    def wait(self) -> None:
        """Wait for the allreduce started by :meth:`prepare_sync`."""
        with torch.profiler.record_function("torchft::local_sgd::wait"):
            if not self._allreduce_work:
                return
            if self._stream is not None:
                assert self._stop_event is not None
                self._stop_event.synchronize()
                self._stop_event = None
            self._allreduce_work = []

    def prepare_sync(self) -> None:
        """Form the pseudo-gradients and start averaging them; does not wait."""
        with torch.profiler.record_function("torchft::local_sgd::prepare_sync"):
            self._save_grads()
            assert not self._allreduce_work
            if self._stream is not None:
                self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream) if self._stream is not None else nullcontext():
                self._average_grads()

    def perform_sync(self) -> bool:
        """Finish the allreduce, vote, and on success take the outer optimizer step."""
        with torch.profiler.record_function("torchft::local_sgd::perform_sync"):
            assert self._allreduce_work
            with torch.cuda.stream(self._stream) if self._stream is not None else nullcontext():
                for w in self._allreduce_work:
                    w.wait()
                if self._stream is not None:
                    self._stop_event = torch.cuda.Event()
                    self._stop_event.record()
            self.wait()
            # remember the local weights, then go back to the last global ones: if the vote
            # fails the fragment stays there and the window is retried
            self._save_local_parameters()
            self.restore_parameters()
            committed = self._manager.should_commit()
            if committed:
                self._set_grads()
                self._outer_optimizer.step()
                self.save_parameters()
                self._merge_parameters()
            self._outer_optimizer.zero_grad()
            self._clear_local_parameters()
            self._grads.clear()
            return committed

    def _average_grads(self) -> None:
        if self.use_bucketization:
            self._allreduce_bucketized()
        else:
            self._allreduce_per_param()

    def _allreduce_per_param(self) -> None:
        for name, _ in self._model_fragment.named_parameters():
            self._allreduce_work.append(self._manager.allreduce(self._grads[name], should_quantize=self.should_quantize))

    def _bucketize_and_allreduce(self, tensors: List[torch.Tensor], bucket_size_bytes: int) -> None:
        """Pack ``tensors`` into flat buffers of at most ``bucket_size_bytes`` and allreduce
        each buffer; results are copied back when the buffer's work completes.  A tensor
        larger than the cap gets a bucket of its own (nothing is ever dropped)."""
        if not tensors:
            return
        dtype, device = tensors[0].dtype, tensors[0].device
        cap = max(1, bucket_size_bytes // tensors[0].element_size())
        i = 0
        while i < len(tensors):
            group: List[torch.Tensor] = [tensors[i]]
            used = tensors[i].numel()
            i += 1
            while i < len(tensors) and used + tensors[i].numel() <= cap:
                group.append(tensors[i])
                used += tensors[i].numel()
                i += 1
            flat = torch.empty(used, dtype=dtype, device=device)
            views: List[Tuple[torch.Tensor, int, int]] = []
            off = 0
            for t in group:
                n = t.numel()
                flat[off : off + n].copy_(t.reshape(-1))
                views.append((t, off, n))
                off += n
            work = self._manager.allreduce(flat, should_quantize=self.should_quantize)

            def unpack(fut: torch.futures.Future, flat=flat, views=views) -> List[torch.Tensor]:
                for t, o, n in views:
                    t.copy_(flat[o : o + n].view_as(t))
                return []

            work.get_future().then(unpack)
            self._allreduce_work.append(work)

    def _allreduce_bucketized(self) -> None:
        grads = list(self._grads.values())
        assert grads, "No gradients to allreduce"
        self._bucketize_and_allreduce(grads, bucket_size_bytes=self.bucket_cap_mb)


def _flat_eligible(fragment: nn.Module, outer: optim.Optimizer) -> bool:
    """Whether a fragment can live in flat buffers: plain tensors of one fp32/bf16 dtype on
    one device, and an outer optimizer that is momentum SGD without damping or decay."""
    params = list(fragment.parameters())
    if not params or not isinstance(outer, optim.SGD) or len(outer.param_groups) != 1:
        return False
    g = outer.param_groups[0]
    if g.get("dampening", 0) != 0 or g.get("weight_decay", 0) != 0 or g.get("maximize", False):
        return False
    p0 = params[0]
    if p0.dtype not in (torch.float32, torch.bfloat16):
        return False
    for p in params:
        if (DTensor is not None and isinstance(p, DTensor)) or p.dtype != p0.dtype or p.device != p0.device:
            return False
    return True


class _FlatDiLoCoFragment(_StreamingDiLoCoFragment):
    """A fragment kept in four flat buffers on the parameters' device: the live weights (the
    module's parameters become views into it), the last global weights, the averaged
    pseudo-gradient and the fp32 outer momentum.

    A synchronisation is then two kernels instead of several passes per parameter:
    :meth:`Manager.allreduce_delta` (with fp8 on a peer-memory process group: difference,
    quantisation, reduction and averaging fused) and :func:`torchft_b200.ops.diloco.outer_step_`
    (momentum, Nesterov step, new backup, blend with the local weights).  The hyperparameters
    are read from the outer optimizer's single param group at every step, so LR schedulers on
    it keep working; its ``momentum_buffer`` state entries are views of the flat momentum, so
    ``outer_optimizer.state_dict()`` is what the per-parameter fragment would give and the two
    layouts can heal each other.  The scheduling and the state-dict key are those of the per-parameter fragment
    (torchft/local_sgd.py:176-560).
    """

    _PAD = 128 * 8  # whole quantisation blocks for every team size up to 8

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        params = [p for _, p in self._model_fragment.named_parameters()]
        dtype, dev = params[0].dtype, params[0].device
        n = sum(p.numel() for p in params)
        padded = (n + self._PAD - 1) // self._PAD * self._PAD
        self._flat_param = torch.zeros(padded, dtype=dtype, device=dev)
        self._flat_backup = torch.zeros(padded, dtype=dtype, device=dev)
        self._flat_grad = torch.zeros(padded, dtype=dtype, device=dev)
        self._flat_momentum = torch.zeros(padded, dtype=torch.float32, device=dev)
        self._layout: List[Tuple[str, nn.Parameter, int, int]] = []
        off = 0
        with torch.no_grad():
            for name, p in self._model_fragment.named_parameters():
                k = p.numel()
                view = self._flat_param[off : off + k].view(p.shape)
                view.copy_(p.data)
                p.data = view
                self.original_parameters[name] = self._flat_backup[off : off + k].view(p.shape)
                self._layout.append((name, p, off, k))
                off += k
        self._publish_momentum()

    def _publish_momentum(self) -> None:
        """The outer optimizer's ``momentum_buffer`` entries are views of the flat momentum, so
        ``outer_optimizer.state_dict()`` carries the momentum exactly as with the per-parameter
        fragment (checkpoints written the reference's way keep working).  A zero buffer is the
        same as torch's "no buffer yet": with dampening 0 the first step gives ``buf = grad``."""
        owned = {id(q) for g in self._outer_optimizer.param_groups for q in g["params"]}
        for _, p, off, k in self._layout:
            if id(p) in owned:
                self._outer_optimizer.state[p]["momentum_buffer"] = self._flat_momentum[off : off + k].view(p.shape)

    def _adopt_momentum(self) -> None:
        """After ``outer_optimizer.load_state_dict`` (which replaces state tensors by copies): take the
        loaded buffers into the flat momentum and publish the views again."""
        with torch.no_grad():
            for _, p, off, k in self._layout:
                buf = self._outer_optimizer.state.get(p, {}).get("momentum_buffer")
                dst = self._flat_momentum[off : off + k]
                if buf is None:
                    dst.zero_()
                elif buf.data_ptr() != dst.data_ptr():
                    dst.copy_(buf.reshape(-1))
        self._publish_momentum()

    def _check_views(self) -> None:
        """``model.to()``, ``load_state_dict(assign=True)`` or a later wrapper can re-point a parameter
        away from the flat buffer; the fused kernels would then silently synchronise stale memory."""
        base, es = self._flat_param.data_ptr(), self._flat_param.element_size()
        for name, p, off, _ in self._layout:
            if p.data_ptr() != base + off * es:
                raise RuntimeError(
                    f"parameter {name!r} no longer lives in its DiLoCo fragment's flat buffer (it was moved or "
                    "re-assigned after DiLoCo was built); build DiLoCo after the last .to()/wrap, or pass "
                    "flat_fragments=False")

    def register_state_dict_fn(self) -> None:
        key = f"StreamingDiLoCoFragment_{self._fragment_id}"

        def load_fn(sd: Dict[str, Any]) -> None:
            # accepts what a per-parameter fragment (here or in the reference) saved, and the older
            # flat layout that carried the momentum under "outer_momentum"
            for name, value in sd["original_parameters"].items():
                if name in self.original_parameters:
                    self.original_parameters[name].copy_(value)
            self._outer_optimizer.load_state_dict(sd["outer_optimizer"])
            if "outer_momentum" in sd:
                self._flat_momentum.copy_(sd["outer_momentum"])
                self._publish_momentum()
            else:
                self._adopt_momentum()

        def save_fn() -> Dict[str, Any]:
            return {
                "outer_optimizer": self._outer_optimizer.state_dict(),
                "original_parameters": {n: t.clone() for n, t in self.original_parameters.items()},
            }

        self._manager.register_state_dict_fn(key, load_fn, save_fn)

    def save_parameters(self) -> None:
        with torch.no_grad():
            self._flat_backup.copy_(self._flat_param)

    def restore_parameters(self) -> None:
        with torch.no_grad():
            self._flat_param.copy_(self._flat_backup)

    def prepare_sync(self) -> None:
        with torch.profiler.record_function("torchft::local_sgd::prepare_sync"), torch.no_grad():
            assert not self._allreduce_work
            self._check_views()
            early = self._fragment_sync_delay > 0
            if early:
                # inner steps go on while the exchange is in flight: take the difference now
                torch.sub(self._flat_backup, self._flat_param, out=self._flat_grad)
            if self._stream is not None:
                self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream) if self._stream is not None else nullcontext():
                if early:
                    work = self._manager.allreduce(self._flat_grad, should_quantize=self.should_quantize)
                else:
                    work = self._manager.allreduce_delta(self._flat_grad, self._flat_backup, self._flat_param,
                                                         should_quantize=self.should_quantize)
                self._allreduce_work.append(work)

    def perform_sync(self) -> bool:
        from .ops.diloco import outer_step_

        with torch.profiler.record_function("torchft::local_sgd::perform_sync"), torch.no_grad():
            assert self._allreduce_work
            with torch.cuda.stream(self._stream) if self._stream is not None else nullcontext():
                for w in self._allreduce_work:
                    w.wait()
                if self._stream is not None:
                    self._stop_event = torch.cuda.Event()
                    self._stop_event.record()
            self.wait()
            committed = self._manager.should_commit()
            if committed:
                g = self._outer_optimizer.param_groups[0]
                outer_step_(self._flat_grad, self._flat_momentum, self._flat_backup, self._flat_param, lr=float(g["lr"]),
                            momentum_coef=float(g.get("momentum", 0.0)), alpha=self._fragment_update_alpha,
                            nesterov=bool(g.get("nesterov", False)), first_step=False)
            else:
                # back to the last global weights; the manager step did not advance, so the window is retried
                self._flat_param.copy_(self._flat_backup)
            return committed


class DiLoCo:
    """(Streaming) DiLoCo as a context manager around the inner optimizer.

    With ``F = len(model_fragments)`` fragments, every ``sync_every / F`` inner steps one
    fragment (``manager.current_step() % F``) is synchronised; its allreduce starts
    ``fragment_sync_delay`` steps earlier.  Requires a manager with
    ``use_async_quorum=False`` (a healing replica must have its weights before it
    computes a pseudo-gradient).  If a window does not commit, the fragment is reset to
    the last global weights and, the manager step not having advanced, retried.

    ``flat_fragments`` keeps every fragment in flat device buffers and synchronises it with
    two fused kernels (see :class:`_FlatDiLoCoFragment`); it needs a momentum-SGD outer
    optimizer without damping or weight decay.  Default: on for CUDA parameters unless ``backup_device`` names
    the host.
    """

    def __init__(
        self,
        manager: Manager,
        model_fragments: List[nn.Module],
        inner_optimizer: optim.Optimizer,
        outer_optimizer: Union[optim.Optimizer, List[optim.Optimizer]],
        sync_every: int,
        backup_device: Optional[torch.device] = None,
        pin_memory: bool = True,
        use_bucketization: bool = False,
        bucket_cap_mb: Optional[int] = None,
        should_quantize: bool = False,
        fragment_sync_delay: int = 0,
        fragment_update_alpha: float = 0.0,
        flat_fragments: Optional[bool] = None,
    ) -> None:
        n = len(model_fragments)
        if isinstance(outer_optimizer, list):
            assert len(outer_optimizer) == n, "The number of outer optimizers must match the number of model fragments"
        if manager._use_async_quorum:
            raise ValueError(
                "Using DiLoCo require synchronous quorum to be enabled. "
                "Ensure that the manager is initialized with use_async_quorum=False"
            )
        if sync_every < n:
            raise ValueError("Only 1 fragment can be syncrhonized at a time")
        if sync_every % n != 0:
            raise ValueError("sync_every must divide the number of fragments")
        self._sync_every: int = sync_every // n
        if fragment_sync_delay >= self._sync_every:
            raise ValueError("Fragment must be synced before it is reduced another time")
        if fragment_update_alpha < 0 or fragment_update_alpha > 1:
            raise ValueError("fragment_update_alpha must be between 0 and 1")

        self._manager = manager
        self._local_step = 0
        self._fragment_sync_delay = fragment_sync_delay
        self._hooks: List[RemovableHandle] = []
        self._local_optimizer = inner_optimizer
        outers = outer_optimizer if isinstance(outer_optimizer, list) else [outer_optimizer] * n
        eligible = all(_flat_eligible(f, o) for f, o in zip(model_fragments, outers))
        if flat_fragments is None:
            # HBM holds the backup next to the weights unless the caller asked for a host backup
            on_gpu = all(p.is_cuda for f in model_fragments for p in f.parameters())
            flat_fragments = eligible and on_gpu and (backup_device is None or backup_device.type == "cuda")
        elif flat_fragments and not eligible:
            raise ValueError("flat_fragments needs plain fp32/bf16 parameters and a plain momentum-SGD outer optimizer")
        self.flat_fragments = bool(flat_fragments)
        fragment_cls = _FlatDiLoCoFragment if self.flat_fragments else _StreamingDiLoCoFragment
        self._fragments: List[_StreamingDiLoCoFragment] = [
            fragment_cls(
                manager,
                frag,
                i,
                math.floor((sync_every / n) * (i + 1)),
                inner_optimizer,
                outer_optimizer[i] if isinstance(outer_optimizer, list) else outer_optimizer,
                sync_every,
                backup_device,
                pin_memory,
                use_bucketization,
                bucket_cap_mb,
                should_quantize,
                fragment_sync_delay,
                fragment_update_alpha,
            )
            for i, frag in enumerate(model_fragments)
        ]
        self._save_parameters()
        for f in self._fragments:
            f.register_state_dict_fn()

    def _save_parameters(self) -> None:
        for f in self._fragments:
            f.save_parameters()

    def _restore_parameters(self) -> None:
        for f in self._fragments:
            f.restore_parameters()

    def __enter__(self) -> "DiLoCo":
        self._hooks.append(self._local_optimizer.register_step_pre_hook(self._step_pre_hook))
        self._hooks.append(self._local_optimizer.register_step_post_hook(self._step_post_hook))
        return self

    def __exit__(self, exc_type: Optional[Type[BaseException]], exc_value: Optional[BaseException],
                 tb: Optional[TracebackType]) -> bool:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        return False

    def _step_pre_hook(self, _o: optim.Optimizer, _a: Tuple[Any, ...], _k: Dict[str, Any]) -> None:
        self._manager.disallow_state_dict_read()

    def _wait(self) -> None:
        for f in self._fragments:
            f.wait()

    def _current_fragment(self) -> int:
        return self._manager.current_step() % len(self._fragments)

    def _step_post_hook(self, _o: optim.Optimizer, _a: Tuple[Any, ...], _k: Dict[str, Any]) -> None:
        self._manager.allow_state_dict_read()
        self._local_step += 1
        if self._local_step == self._sync_every - self._fragment_sync_delay:
            # quorum (and, for a behind replica, healing) happens here, synchronously
            self._manager.start_quorum()
            frag = self._current_fragment()
            logger.info(f"Preparing fragment={frag} step={self._local_step}")
            self._fragments[frag].prepare_sync()
        if self._local_step < self._sync_every:
            return
        assert self._local_step == self._sync_every, f"{self._local_step=} exceeded {self._sync_every=}"
        frag = self._current_fragment()
        logger.info(f"Syncing fragment={frag} step={self._local_step} manager_step={self._manager.current_step()}")
        self._fragments[frag].perform_sync()
        self._local_step = 0
