"""Fault-tolerant HSDP trainer for the Llama engine.

Sharding (inside a replica group) is FSDP-style over flat per-layer units: every rank
owns ``1/shard_size`` of each unit as a bf16 working shard plus fp32 master weights and
AdamW moments.  Full (gathered) bf16 units stay resident between forward and backward
(B200 has the HBM for it), so each unit is all-gathered once per step, prefetched one
unit ahead on a communication stream.  Gradients are produced into double-buffered
full units, reduce-scattered to shards as soon as a unit's backward ends, then averaged
over the replica dimension through ``Manager.allreduce`` -- the only place the
fault-tolerant world size appears.  ``Manager.should_commit`` gates the optimizer step.

The replica dimension mirrors what the reference obtains by giving FSDP2 a device mesh
whose replicate dimension is a ``ManagedProcessGroup`` (torchft/device_mesh.py:307-340).
"""

from __future__ import annotations

import math
import os
from typing import Dict, List, Optional

import torch

from ..models.llama import LlamaConfig, LlamaEngine, init_unit_
from ..ops import kernels as K
from .shard_comm import LocalShardComm, ShardComm


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def shard_pieces(offset: int, numel: int, shard_numel: int) -> List[tuple]:
    """The pieces of the element range ``[offset, offset + numel)`` of a flat unit that is sharded evenly in shards of
    ``shard_numel`` elements: ``(owner rank, offset inside the owner's shard, offset inside the unit, elements)``, cut
    at the shard boundaries."""
    out, a, end = [], offset, offset + numel
    while a < end:
        owner = a // shard_numel
        b = min(end, (owner + 1) * shard_numel)
        out.append((owner, a - owner * shard_numel, a, b - a))
        a = b
    return out


class ShardedLlamaTrainer:
    """Llama trainer on the explicit engine with FSDP-style sharding inside the replica group and an optional managed
    replica dimension.  Parameters, gradients and AdamW state live as one shard per rank and unit (a unit is the
    embedding, one decoder layer, or the head); ``shard_comm`` gathers a unit's parameters ahead of its GEMMs and
    reduce-scatters its gradients; with ``manager`` the shard-sized gradients are averaged over the replica groups and
    the optimizer runs only when the step commits.  ``train_step(tokens, targets)`` is one complete step and returns
    the loss; ``state_dict()`` / ``load_state_dict()`` expose this rank's shards for healing and checkpoints."""

    def __init__(
        self,
        cfg: LlamaConfig,
        batch: int,
        seq_len: int,
        device: torch.device,
        shard_comm: Optional[ShardComm] = None,
        manager=None,
        lr: float = 3e-4,
        betas=(0.9, 0.95),
        eps: float = 1e-8,
        weight_decay: float = 0.1,
        max_grad_norm: float = 1.0,
        seed: int = 0,
        attention=None,
        logit_chunks: int = 4,
        replica_alloc=None,
        fused_reduce_scatter: bool = True,
        fused_all_gather: Optional[bool] = None,
        wgrad_stream: Optional[bool] = None,
        save_norms: Optional[bool] = None,
    ):
        self.cfg, self.device = cfg, device
        self.comm = shard_comm or LocalShardComm()
        self.manager = manager
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.opt_step = 0
        ws, rank = self.comm.size, self.comm.rank
        self.cuda = device.type == "cuda"
        U = cfg.n_units
        self.unit_numel = [cfg.unit_numel(u) for u in range(U)]
        self.shard_numel = [_round_up(n, ws * 8) // ws for n in self.unit_numel]
        self.full_numel = [s * ws for s in self.shard_numel]

        bf, f32 = torch.bfloat16, torch.float32
        A = self.comm.alloc
        # shards that peers of the shard group read (all-gather sources) come from the shard
        # communicator; gradient shards are what the replica dimension reduces, so they come
        # from the replica group's allocator when it has one (in-place peer-memory allreduce)
        # Every kind of per-rank state is ONE allocation with the units as views: the optimizer and the gradient norm
        # are then single launches over the whole model, and a peer that heals from this rank maps three allocations
        # (master weights and the two AdamW moments) instead of three per unit.
        def carve(flat: torch.Tensor) -> List[torch.Tensor]:
            out, off = [], 0
            for n in self.shard_numel:
                out.append(flat[off : off + n])
                off += n
            return out

        total = sum(self.shard_numel)
        self.p_flat = A(total, bf, device)
        self.p_shard = carve(self.p_flat)
        self.g_flat = replica_alloc(total, bf) if replica_alloc is not None else torch.empty(total, dtype=bf, device=device)
        self.g_shard = carve(self.g_flat)
        self.master_flat = torch.empty(total, dtype=f32, device=device)
        self.m_flat = torch.zeros(total, dtype=f32, device=device)
        self.v_flat = torch.zeros(total, dtype=f32, device=device)
        self.master, self.m, self.v = carve(self.master_flat), carve(self.m_flat), carve(self.v_flat)
        if ws == 1:
            self.p_full = self.p_shard
            self._g_bufs: Dict[int, List[torch.Tensor]] = {}
        else:
            self.p_full = [torch.empty(n, dtype=bf, device=device) for n in self.full_numel]
            sizes = sorted(set(self.full_numel))
            self._g_bufs = {s: [A(s, bf, device) for _ in range(2 if self.full_numel.count(s) > 1 else 1)] for s in sizes}
        self._g_slot = [0] * U
        cnt: Dict[int, int] = {}
        for u in range(U):
            s = self.full_numel[u]
            self._g_slot[u] = cnt.get(s, 0) % 2
            cnt[s] = cnt.get(s, 0) + 1

        # deterministic init: every rank generates the full unit, keeps its slice
        for u in range(U):
            if ws == 1:
                init_unit_(cfg, u, self.p_full[u][: self.unit_numel[u]], seed)
                self.p_full[u][self.unit_numel[u]:].zero_()
            else:
                full = self.p_full[u]
                full.zero_()
                init_unit_(cfg, u, full[: self.unit_numel[u]], seed)
                n = self.shard_numel[u]
                self.p_shard[u].copy_(full[rank * n : (rank + 1) * n])
            self.master[u].copy_(self.p_shard[u].float())

        # communication (shard-group and replica-dimension) runs beside compute
        self.comm_stream = (
            torch.cuda.Stream(device=device, priority=-1) if self.cuda and (ws > 1 or manager is not None) else None
        )
        self._ag_event: List[Optional[torch.cuda.Event]] = [None] * U
        self._rs_event: Dict[int, Optional[torch.cuda.Event]] = {}
        self._gathered = [ws == 1] * U
        self._works: List = []
        # FTB200_TIMELINE=1: bracket every point at which the compute stream waits for the communication stream with
        # CUDA events; `exposed_comm_ms()` then says how much of the gathers and reductions was not hidden
        self._timeline = self.cuda and os.environ.get("FTB200_TIMELINE", "0") == "1"
        self._stalls: Dict[str, List[tuple]] = {"all_gather": [], "grad_buffer": [], "tail": []}
        self.sumsq = torch.zeros(1, dtype=f32, device=device)
        self.clip = torch.ones(1, dtype=f32, device=device)
        self.grad_norm = torch.zeros(1, dtype=f32, device=device)
        # GEMM-fused reduce-scatter: the weight-gradient GEMMs store their tiles straight into the
        # shard owners' staging areas (the double-buffered full-unit buffers, viewed as
        # [world, shard]); what is left of the reduce-scatter is a team round and a local sum.
        self.fused_rs = bool(
            fused_reduce_scatter and ws > 1 and self.cuda and getattr(self.comm, "supports_fused_scatter", False)
            and K.GEMM_IMPL == "2cta" and logit_chunks == 1
        )
        self._fused_fields: Dict[int, object] = {}
        self._vec_tmp: Dict[str, torch.Tensor] = {}
        # GEMM-fused all-gather (FTB200_AG_FUSED=1 or fused_all_gather=True): the decoder layers and the head are not
        # gathered ahead of time; each forward GEMM pulls its own weight out of the shard owners' memory while it
        # multiplies.  What is left for the communication stream at the start of a step is the embedding unit and
        # one small copy kernel for the norm weights of all units.
        if fused_all_gather is None:
            fused_all_gather = os.environ.get("FTB200_AG_FUSED", "0") == "1"
        self.fused_ag = bool(
            fused_all_gather and ws > 1 and self.cuda and getattr(self.comm, "supports_fused_scatter", False)
            and K.GEMM_IMPL == "2cta"
        )
        self._params_event: Optional[torch.cuda.Event] = None
        self._ga_fields: Dict[int, object] = {}
        self._ga_units: List[int] = []
        if self.fused_ag:
            self._build_gather_fields()
        if self.fused_rs:
            for bufs in self._g_bufs.values():
                for b in bufs:
                    b.zero_()  # padding of the last shard is never written again
        self.engine = LlamaEngine(
            cfg, batch, seq_len, device, self._param_unit, self._grad_unit, self._before_unit, self._grad_done,
            attention=attention, logit_chunks=logit_chunks, grad_fields=self._grad_fields if self.fused_rs else None,
            grad_scale=1.0 / ws,  # the shard group sums its gradients: scale so that the sum is the mean over the group
            fwd_fields=self._fwd_fields if self.fused_ag else None,
            # Weight gradients on a second stream pay off when the backward pass has the GPU to itself (-2 % step
            # time on one GPU); next to the replica dimension's allreduce kernels they measured 3 % slower on two
            # groups, so by default they are used only without a shard group and without a manager.  A job that
            # knows it runs a single replica group passes True.
            wgrad_stream=(ws == 1 and manager is None) if wgrad_stream is None else bool(wgrad_stream),
            save_norms=save_norms,
        )
        self._mark_params_written()

    # ---- unit plumbing -------------------------------------------------------------------
    def _param_unit(self, u: int) -> torch.Tensor:
        return self.p_full[u][: self.unit_numel[u]]

    def _grad_buf(self, u: int) -> torch.Tensor:
        if self.comm.size == 1:
            return self.g_shard[u]
        return self._g_bufs[self.full_numel[u]][self._g_slot[u] % len(self._g_bufs[self.full_numel[u]])]

    def _grad_unit(self, u: int) -> torch.Tensor:
        return self._grad_buf(u)[: self.unit_numel[u]]

    def _mark_params_written(self) -> None:
        """The parameter shards were just written on the current stream (optimizer step, state load, init): the
        communication stream must not offer them to the peers before that work is done."""
        if self.comm_stream is not None and self.comm.size > 1:
            ev = torch.cuda.Event()
            ev.record()
            self._params_event = ev

    def _build_gather_fields(self) -> None:
        from ..checkpointing.p2p_transport import _seg_table

        ws = self.comm.size
        max_rows = 0
        vec_segs = []
        for u in range(1, self.cfg.n_units):
            fields = self.cfg.unit_fields(u)
            if not all(K.GatherField.supported(shape, self.shard_numel[u]) for _, shape in fields if len(shape) == 2):
                continue
            max_rows = max(max_rows, max(shape[0] for _, shape in fields if len(shape) == 2))
            self._ga_units.append(u)
        if not self._ga_units:
            self.fused_ag = False
            return
        self._ga_sync = torch.zeros(1 + max_rows // 128, dtype=torch.int32, device=self.device)

        class _F:
            pass

        for u in self._ga_units:
            f = _F()
            f.matrices = []
            peers = self.comm.stage_peers(self.p_shard[u])
            n = self.shard_numel[u]
            off = 0
            for name, shape in self.cfg.unit_fields(u):
                numel = math.prod(shape)
                local = self.p_full[u][off : off + numel].view(*shape)
                if len(shape) == 2:
                    g = K.GatherField(local, peers, ws, n, off, self._ga_sync)
                    setattr(f, name, g)
                    f.matrices.append(g)
                else:
                    setattr(f, name, local)
                    # norm weights travel in one copy kernel per step: split at shard boundaries
                    for owner, in_shard, in_unit, count in shard_pieces(off, numel, n):
                        vec_segs.append((int(peers[owner]) + in_shard * 2, self.p_full[u].data_ptr() + in_unit * 2, count * 2))
                off += numel
            self._ga_fields[u] = f
        if any(nb % 16 or src % 16 or dst % 16 for src, dst, nb in vec_segs):
            raise ValueError("norm-weight fields must be 16-byte aligned pieces for the fused all-gather")
        self._ga_vec_table = _seg_table(vec_segs, self.device)
        self._ga_vec_n = len(vec_segs)
        self._ga_vec_bytes = sum(s[2] for s in vec_segs)

    def _fwd_fields(self, u: int):
        return self._ga_fields.get(u)

    def _issue_fused_prologue(self) -> None:
        """Start of a step with the GEMM-fused all-gather: on the communication stream, after this rank's parameter
        writes, gather the embedding unit (its rounds also tell every rank that all shards of all units are final)
        and copy the norm weights of the fused units; the layers' matrices are marked as not yet gathered."""
        with torch.cuda.stream(self.comm_stream):
            if self._params_event is not None:
                self.comm_stream.wait_event(self._params_event)
            self.comm.all_gather(self.p_shard[0], self.p_full[0])
            self.comm.copy_segments(self._ga_vec_table, self._ga_vec_n, self._ga_vec_bytes)
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
        self._ag_event[0] = ev
        self._gathered[0] = True
        for u in self._ga_units:
            self._gathered[u] = True
            for g in self._ga_fields[u].matrices:
                g.pending = True

    def _issue_all_gather(self, u: int) -> None:
        if self._gathered[u] or u >= self.cfg.n_units:
            return
        if self.fused_ag and u == 0:
            self._issue_fused_prologue()
            return
        if self.comm_stream is not None:
            with torch.cuda.stream(self.comm_stream):
                if self._params_event is not None:
                    self.comm_stream.wait_event(self._params_event)
                self.comm.all_gather(self.p_shard[u], self.p_full[u])
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
            self._ag_event[u] = ev
        else:
            self.comm.all_gather(self.p_shard[u], self.p_full[u])
        self._gathered[u] = True

    def _before_unit(self, u: int, backward: bool) -> None:
        if self.comm.size == 1:
            return
        if not backward:
            self._issue_all_gather(u)
            ev = self._ag_event[u]
            if ev is not None:
                self._wait_timed("all_gather", lambda: torch.cuda.current_stream().wait_event(ev))
                self._ag_event[u] = None
            if u + 1 < self.cfg.n_units:
                self._issue_all_gather(u + 1)
        else:
            # the gradient buffer about to be written may still feed an earlier reduce-scatter
            key = self._grad_buf(u).data_ptr()
            ev = self._rs_event.pop(key, None)
            if ev is not None:
                self._wait_timed("grad_buffer", lambda: torch.cuda.current_stream().wait_event(ev))

    def _grad_fields(self, u: int):
        """Scatter targets for the matrices of unit ``u`` (None for the embedding unit, whose
        gradient is built by atomics in a local buffer and reduce-scattered the plain way)."""
        if u == 0:
            return None
        f = self._fused_fields.get(u)
        if f is None:

            class _F:
                pass

            f = _F()
            f.vectors = []
            stage = self._grad_buf(u)
            peers = self.comm.stage_peers(stage)
            off = 0
            for name, shape in self.cfg.unit_fields(u):
                field = K.ScatterField(peers, self.comm.size, self.comm.rank, self.shard_numel[u], off, shape)
                if len(shape) == 2:
                    setattr(f, name, field)
                else:
                    tmp = self._vec_tmp.get(name)
                    if tmp is None:
                        tmp = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
                        self._vec_tmp[name] = tmp
                    setattr(f, name, tmp)
                    f.vectors.append((tmp, field))
                off += math.prod(shape)
            self._fused_fields[u] = f
        return f

    def _grad_done(self, u: int) -> None:
        ws = self.comm.size
        if ws > 1 and self.fused_rs and u > 0:
            f = self._grad_fields(u)
            for tmp, field in f.vectors:
                K.scatter_to_stage(tmp, field)
            buf = self._grad_buf(u)
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self.comm.reduce_stage(buf, self.g_shard[u])
                self._replica_allreduce(u)
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
            self._rs_event[buf.data_ptr()] = ev
        elif ws > 1:
            buf = self._grad_buf(u)
            pad = self.full_numel[u] - self.unit_numel[u]
            if pad:
                buf[self.unit_numel[u]:].zero_()
            if self.comm_stream is not None:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm_stream):
                    self.comm.reduce_scatter(buf, self.g_shard[u])
                    self._replica_allreduce(u)
                    ev = torch.cuda.Event()
                    ev.record(self.comm_stream)
                self._rs_event[buf.data_ptr()] = ev
            else:
                self.comm.reduce_scatter(buf, self.g_shard[u])
                self._replica_allreduce(u)
        elif self.manager is not None and self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                self._replica_allreduce(u)
        else:
            self._replica_allreduce(u)

    def _replica_allreduce(self, u: int) -> None:
        if self.manager is not None:
            self._works.append(self.manager.allreduce(self.g_shard[u]))

    # ---- public step ---------------------------------------------------------------------
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        if self.cuda and self.comm.size > 1:
            # head/embedding units use single gradient buffers: order against last step's readers
            pass
        loss = self.engine.forward(tokens, targets, train=True)
        self.engine.backward(tokens)
        return loss

    def _finish_comm(self) -> None:
        for w in self._works:
            w.wait()
        self._works.clear()
        if self.comm_stream is not None:
            self._wait_timed("tail", lambda: torch.cuda.current_stream().wait_stream(self.comm_stream))
        self._rs_event.clear()

    def _wait_timed(self, kind: str, wait) -> None:
        if not self._timeline:
            wait()
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        wait()
        b.record()
        self._stalls[kind].append((a, b))

    def exposed_comm_ms(self, reset: bool = True) -> Dict[str, float]:
        """With ``FTB200_TIMELINE=1``: milliseconds the compute stream spent, since the last call, waiting for the
        communication stream -- for a unit's all-gather before its first GEMM, for a gradient buffer still being
        reduced, and for the tail of the reductions after the backward pass.  Synchronises the device."""
        torch.cuda.synchronize(self.device)
        out = {k: float(sum(a.elapsed_time(b) for a, b in v)) for k, v in self._stalls.items()}
        if reset:
            for v in self._stalls.values():
                v.clear()
        return out

    def optimizer_step(self) -> None:
        self.opt_step += 1
        self.sumsq.zero_()
        K.sumsq_(self.g_flat, self.sumsq)
        self.comm.all_reduce_sum_(self.sumsq)
        K.clip_coef_(self.sumsq, self.max_grad_norm, self.clip, self.grad_norm)
        b1, b2 = self.betas
        K.adamw_(self.master_flat, self.m_flat, self.v_flat, self.g_flat, self.p_flat, self.lr, b1, b2, self.eps, self.wd,
                 self.opt_step, self.clip)
        if self.comm.size > 1:
            self._gathered = [False] * self.cfg.n_units
            self._mark_params_written()

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One fault-tolerant step: quorum, forward/backward with overlapped gradient
        reduction, commit vote, optimizer step."""
        if self.manager is not None:
            self.manager.start_quorum()
        loss = self.forward_backward(tokens, targets)
        self._finish_comm()
        self._check_shard_team()
        if self.manager is None or self.manager.should_commit():
            self.optimizer_step()
        return loss

    def _check_shard_team(self) -> None:
        """A shard-group kernel (all-gather, reduce-scatter, the GEMM-fused reduce stage) that ran into its
        deadline or an abort returns with stale parameters or partial gradients behind it and says so only in
        the team's status word.  Read it before the vote: with a manager the step is declined (and the error
        latched, so the healthy groups do not average this group's gradients in); without one it raises."""
        team = getattr(self.comm, "team", None)
        if team is None:
            return
        code = team.status()
        if code == 0:
            return
        from ..ops import _native as N
        from .team import TeamError

        err = TeamError(f"shard-group collective failed: {N.STATUS.get(code, code)}")
        if self.manager is None:
            raise err
        self.manager.report_error(err)

    def invalidate_gathered(self, units) -> None:
        """The shards of ``units`` were rewritten outside :meth:`optimizer_step`: gather them
        again before their next use."""
        if self.comm.size > 1:
            for u in units:
                self._gathered[u] = False
            self._mark_params_written()  # (the caller wrote the shards on the current stream)

    # ---- state dict (heal / durable checkpoints) -------------------------------------------
    def state_dict(self) -> Dict[str, object]:
        return {
            "opt_step": self.opt_step,
            "master": self.master,
            "m": self.m,
            "v": self.v,
        }

    def load_state_dict(self, sd: Dict[str, object]) -> None:
        self.opt_step = int(sd["opt_step"])
        for u in range(self.cfg.n_units):
            self.master[u].copy_(sd["master"][u])
            self.m[u].copy_(sd["m"][u])
            self.v[u].copy_(sd["v"][u])
            self.p_shard[u].copy_(self.master[u].to(torch.bfloat16))
        if self.comm.size > 1:
            self._gathered = [False] * self.cfg.n_units
            self._mark_params_written()
