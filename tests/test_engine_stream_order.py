"""Ordering of the engine's two backward streams, checked without a GPU.

The weight-gradient GEMMs of the backward pass run on a stream of their own, ordered against the main stream by
events per operand workspace.  A missing wait is a data race that a GPU test may never show, so this test runs the
backward pass on CPU with stand-ins for CUDA streams and events, records which stream every kernel call was issued
on and which buffers it reads and writes, derives the happens-before relation from the streams' program order and
the recorded event waits, and requires every pair of conflicting accesses from different streams to be ordered.
"""
import contextlib
import itertools

import pytest
import torch

from torchft_b200.models import llama as L
from torchft_b200.ops import kernels as K
from torchft_b200.parallel.hsdp import ShardedLlamaTrainer


class _Stream:
    _ids = itertools.count()

    def __init__(self, *a, **k):
        self.id = next(self._ids)
        self.clock = {}  # stream id -> number of that stream's operations known to precede this stream's next one
        self.n_ops = 0

    def _merge(self, other_clock):
        for k, v in other_clock.items():
            if v > self.clock.get(k, 0):
                self.clock[k] = v

    def wait_event(self, ev):
        if ev.snapshot is not None:
            self._merge(ev.snapshot)

    def wait_stream(self, other):
        snap = dict(other.clock)
        snap[other.id] = other.n_ops
        self._merge(snap)

    def synchronize(self):
        pass


class _Event:
    def __init__(self, *a, **k):
        self.snapshot = None

    def record(self, stream=None):
        s = stream if stream is not None else _Cuda.current
        snap = dict(s.clock)
        snap[s.id] = s.n_ops
        self.snapshot = snap


class _Cuda:
    main = None
    current = None


@contextlib.contextmanager
def _stream_ctx(s):
    prev = _Cuda.current
    _Cuda.current = s if s is not None else prev
    try:
        yield
    finally:
        _Cuda.current = prev


def _span(t):
    """(storage, first byte, last byte + 1) of a contiguous tensor (for a scatter target: of its staging buffer)."""
    if hasattr(t, "peers"):
        t = t.peers.tensor
    es = t.element_size()
    lo = t.storage_offset() * es
    return (t.untyped_storage().data_ptr(), lo, lo + t.numel() * es)


class _Log:
    def __init__(self):
        self.ops = []

    def add(self, name, reads, writes):
        s = _Cuda.current
        s.n_ops += 1
        clock = dict(s.clock)
        clock[s.id] = s.n_ops  # this operation is number n_ops on its stream
        self.ops.append((name, s.id, s.n_ops, clock, [_span(t) for t in reads if t is not None],
                         [_span(t) for t in writes if t is not None]))


def _overlap(a, b):
    return a[0] == b[0] and a[1] < b[2] and b[1] < a[2]


def _ordered(first, second):
    """`first` happens before `second` (different streams): second's clock has seen first's position."""
    _, sid, pos, _, _, _ = first
    return second[3].get(sid, 0) >= pos


def _check(log):
    races = []
    for i, a in enumerate(log.ops):
        for b in log.ops[i + 1:]:
            if a[1] == b[1]:
                continue  # same stream: program order
            conflict = any(_overlap(w, x) for w in a[5] for x in b[4] + b[5]) or any(_overlap(w, x) for w in b[5] for x in a[4])
            if conflict and not _ordered(a, b):
                races.append((a[0], b[0]))
    return races


@pytest.fixture
def fake_cuda(monkeypatch):
    main = _Stream()
    _Cuda.main = _Cuda.current = main
    monkeypatch.setattr(torch.cuda, "Stream", _Stream)
    monkeypatch.setattr(torch.cuda, "Event", _Event)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a, **k: _Cuda.current)
    monkeypatch.setattr(torch.cuda, "stream", _stream_ctx)
    yield main
    _Cuda.main = _Cuda.current = None


def _instrument(monkeypatch, log):
    def wrap(name, fn, reads, writes):
        def inner(*a, **k):
            log.add(name, reads(*a, **k), writes(*a, **k))
            return fn(*a, **k)

        monkeypatch.setattr(K, name, inner)

    wrap("linear_wgrad", K.linear_wgrad, lambda dy, x, out=None, **k: [dy, x], lambda dy, x, out=None, **k: [out])
    wrap("linear_dgrad", K.linear_dgrad, lambda dy, w, out=None, **k: [dy, w], lambda dy, w, out=None, **k: [out])
    wrap("rmsnorm_fwd", K.rmsnorm_fwd,
         lambda x, w, eps=1e-5, res=None, h_out=None, out=None, rstd=None, **k: [x, w, res],
         lambda x, w, eps=1e-5, res=None, h_out=None, out=None, rstd=None, **k: [h_out, out, rstd])
    wrap("rmsnorm_bwd", K.rmsnorm_bwd,
         lambda dy, x, w, rstd, dres=None, dx=None, dw=None, **k: [dy, x, w, rstd, dres],
         lambda dy, x, w, rstd, dres=None, dx=None, dw=None, **k: [dx, dw])
    wrap("swiglu_bwd", K.swiglu_bwd, lambda ds, gu, dgu=None: [ds, gu], lambda ds, gu, dgu=None: [dgu])
    wrap("rope_", K.rope_, lambda buf, *a, **k: [buf], lambda buf, *a, **k: [buf])
    wrap("embedding_bwd", K.embedding_bwd, lambda tok, dout, dtable: [dout], lambda tok, dout, dtable: [dtable])


@pytest.mark.parametrize("save_norms", [False, True])
def test_backward_streams_are_ordered(monkeypatch, fake_cuda, save_norms):
    cfg, B, S = L.LLAMA_TINY, 2, 16
    dev = torch.device("cpu")
    log = _Log()
    done_units = []
    tr = ShardedLlamaTrainer(cfg, B, S, dev, logit_chunks=1, seed=3, save_norms=save_norms)
    eng = tr.engine
    # what a sharding layer's hook does with a finished unit: read its whole gradient buffer (reduce-scatter)
    eng.grad_done = lambda u: (done_units.append((u, _Cuda.current.id)), log.add(f"grad_done[{u}]", [tr._grad_unit(u)], []))
    # switch the second stream on by hand (the engine only creates it on a CUDA device)
    eng.wstream = _Stream()
    eng._w_events, eng._w_last = {}, {}
    # the library attention of the CPU path: one op that reads dout and writes the packed dQKV workspace
    orig_attn_bwd = eng.attn.backward

    def attn_bwd(layer, dout, batch, seq, dqkv):
        log.add("attention.backward", [dout], [dqkv])
        return orig_attn_bwd(layer, dout, batch, seq, dqkv)

    monkeypatch.setattr(eng.attn, "backward", attn_bwd)
    _instrument(monkeypatch, log)
    tokens = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(1))
    targets = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(2))
    loss = tr.forward_backward(tokens, targets)
    assert torch.isfinite(loss)

    on_w = [o for o in log.ops if o[1] == eng.wstream.id]
    assert sum(o[0] == "linear_wgrad" for o in on_w) == 4 * cfg.n_layers  # the layers' weight gradients moved over
    assert [u for u, sid in done_units if sid == eng.wstream.id] == list(range(cfg.n_layers, 0, -1))
    assert _check(log) == []
    # after the backward pass the main stream has seen everything the second stream did
    assert fake_cuda.clock.get(eng.wstream.id, 0) == eng.wstream.n_ops

    # the checker itself: without the waits before a workspace is overwritten it must report races
    monkeypatch.setattr(eng, "_before_overwrite", lambda *names: None)
    n_before = len(log.ops)
    tr.forward_backward(tokens, targets)
    broken = _Log()
    broken.ops = log.ops[n_before:]
    assert _check(broken) != []


def test_shared_norm_gradient_staging_is_not_overwritten_before_the_hook_read_it(monkeypatch, fake_cuda):
    """A sharding layer may hand out the same small staging tensors for the norm-weight gradients of every unit and
    read them in its ``grad_done`` hook (which the engine runs on the second stream): the next unit's norm backward
    on the main stream has to wait for that hook."""
    cfg, B, S = L.LLAMA_TINY, 2, 16
    log = _Log()
    tr = ShardedLlamaTrainer(cfg, B, S, torch.device("cpu"), logit_chunks=1, seed=3)
    eng = tr.engine
    staging = {n: torch.zeros(cfg.dim, dtype=torch.bfloat16) for n in ("attn_norm", "ffn_norm")}

    def fields(u):
        if u == 0 or u == cfg.n_layers + 1:
            return None
        f = L._Fields(tr._grad_unit(u), cfg.unit_fields(u))
        f.attn_norm, f.ffn_norm = staging["attn_norm"], staging["ffn_norm"]
        return f

    eng.grad_fields = fields
    eng.grad_done = lambda u: log.add(f"grad_done[{u}]", [tr._grad_unit(u)] + (list(staging.values()) if 0 < u <= cfg.n_layers else []), [])
    eng.wstream = _Stream()
    eng._w_events, eng._w_last = {}, {}
    monkeypatch.setattr(eng.attn, "backward", lambda layer, dout, batch, seq, dqkv: (log.add("attention.backward", [dout], [dqkv]), dqkv.zero_()))
    _instrument(monkeypatch, log)
    tokens = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(1))
    tr.forward_backward(tokens, tokens)
    assert _check(log) == []


class _LoggingShardComm:
    """A shard group of two as seen from rank 0, in one process: the collectives copy locally and log what they
    read and write on the stream they are issued on."""

    rank, size = 0, 2
    supports_fused_scatter = False

    def __init__(self, log):
        self.log = log

    def alloc(self, numel, dtype, device):
        return torch.zeros(numel, dtype=dtype, device=device)

    def all_gather(self, shard, full):
        self.log.add("all_gather", [shard], [full])
        n = shard.numel()
        full[:n].copy_(shard)
        full[n:2 * n].copy_(shard)

    def reduce_scatter(self, full, shard):
        self.log.add("reduce_scatter", [full], [shard])
        shard.copy_(full[: shard.numel()])

    def all_reduce_sum_(self, t):
        self.log.add("all_reduce_sum", [t], [t])

    def barrier(self):
        pass

    def shutdown(self):
        pass


def test_sharded_trainer_streams_are_ordered(monkeypatch, fake_cuda):
    """The sharded trainer's own stream logic on a shard group of two: parameter gathers one unit ahead on the
    communication stream, gradient buffers shared by alternating units, reduce-scatters behind the backward pass,
    the optimizer's parameter writes against the next step's gathers.  Two steps, so that the hand-over from one
    step to the next is part of the check."""
    cfg, B, S = L.LLAMA_TINY, 2, 16
    log = _Log()
    comm = _LoggingShardComm(log)
    tr = ShardedLlamaTrainer(cfg, B, S, torch.device("cpu"), shard_comm=comm, logit_chunks=1, seed=3, fused_reduce_scatter=False)
    assert tr.comm_stream is None and not tr.fused_rs and not tr.fused_ag
    # what the constructor does on a CUDA device
    tr.cuda = True
    tr.comm_stream = _Stream()
    tr._gathered = [False] * cfg.n_units
    tr._mark_params_written()
    log.ops.clear()
    _instrument(monkeypatch, log)

    def wrap(name, reads, writes):
        fn = getattr(K, name)

        def inner(*a, **k):
            log.add(name, reads(*a, **k), writes(*a, **k))
            return fn(*a, **k)

        monkeypatch.setattr(K, name, inner)

    wrap("linear_fwd", lambda x, w, out=None: [x, w], lambda x, w, out=None: [out])
    wrap("linear_swiglu_fwd", lambda x, w, gu, s: [x, w], lambda x, w, gu, s: [gu, s])
    wrap("embedding_fwd", lambda tok, table, out=None: [table], lambda tok, table, out=None: [out])
    wrap("cross_entropy_", lambda logits, *a, **k: [logits], lambda logits, *a, loss=None, **k: [logits, loss])
    wrap("sumsq_", lambda x, out: [x], lambda x, out: [out])
    wrap("adamw_", lambda master, m, v, grad, param_lp, *a, **k: [grad], lambda master, m, v, grad, param_lp, *a, **k: [master, m, v, param_lp])
    monkeypatch.setattr(tr.engine.attn, "backward",
                        lambda layer, dout, batch, seq, dqkv: (log.add("attention.backward", [dout], [dqkv]), dqkv.zero_()))
    tokens = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(1))
    for _ in range(2):
        loss = tr.train_step(tokens, tokens)
    assert torch.isfinite(loss)
    on_comm = [o[0] for o in log.ops if o[1] == tr.comm_stream.id]
    assert on_comm.count("all_gather") == 2 * cfg.n_units and on_comm.count("reduce_scatter") == 2 * cfg.n_units
    assert _check(log) == []

    # the checker sees the race that the wait for the parameter writes prevents: drop it and run another step
    tr._mark_params_written = lambda: None
    tr._params_event = None
    n_before = len(log.ops)
    tr.train_step(tokens, tokens)
    tr.train_step(tokens, tokens)
    broken = _Log()
    broken.ops = log.ops[n_before:]
    assert any("adamw_" in pair and "all_gather" in pair for pair in _check(broken))


class _Peers(list):
    """Stands in for the ctypes array of peer pointers; remembers the local tensor the pointers belong to."""

    def __init__(self, tensor, world):
        super().__init__([tensor.data_ptr()] * world)
        self.tensor = tensor


class _FusedLoggingShardComm(_LoggingShardComm):
    supports_fused_scatter = True

    def stage_peers(self, t):
        return _Peers(t, self.size)

    def reduce_stage(self, stage, shard):
        self.log.add("reduce_stage", [stage], [shard])

    def copy_segments(self, table, nsegs, total_bytes, ctas=4):
        self.log.add("copy_segments", [self.trainer.p_flat], [self.trainer.p_full[u] for u in self.trainer._ga_units])


@pytest.mark.parametrize("wgrad_stream", [False, True])
def test_sharded_trainer_streams_are_ordered_with_the_fused_collectives(monkeypatch, fake_cuda, wgrad_stream):
    """The same check with the reduce-scatter fused into the weight-gradient GEMMs (which then write the staging
    buffers that the communication stream reduces) and the all-gather fused into the forward GEMMs (which then read
    the shard buffers that the optimizer writes and fill the gathered units themselves)."""
    cfg, B, S = L.LLAMA_TINY, 2, 16
    log = _Log()
    comm = _FusedLoggingShardComm(log)
    tr = ShardedLlamaTrainer(cfg, B, S, torch.device("cpu"), shard_comm=comm, logit_chunks=1, seed=3, fused_reduce_scatter=False)
    comm.trainer = tr
    tr.cuda = True
    tr.comm_stream = _Stream()
    tr._gathered = [False] * cfg.n_units
    # what the constructor does on a CUDA device when both fusions are on
    tr.fused_rs = True
    tr.engine.grad_fields = tr._grad_fields
    tr.fused_ag = True
    tr._build_gather_fields()
    assert tr._ga_units == list(range(1, cfg.n_units))
    tr.engine.fwd_fields = tr._fwd_fields
    if wgrad_stream:  # three streams: main, weight gradients, communication
        tr.engine.wstream = _Stream()
        tr.engine._w_events, tr.engine._w_last = {}, {}
    tr._mark_params_written()
    log.ops.clear()
    _instrument(monkeypatch, log)

    def wrap(name, reads, writes, replace=None):
        fn = replace or getattr(K, name)

        def inner(*a, **k):
            log.add(name, reads(*a, **k), writes(*a, **k))
            return fn(*a, **k)

        monkeypatch.setattr(K, name, inner)

    def gather_gemm(x, w, out, aux=None):
        K.gemm(x, w.local, False, False, out=out)
        if aux is not None:
            K.swiglu_fwd(out, out=aux)
        w.pending = False

    wrap("gemm_gather", lambda x, w, out, aux=None: [x, w.peers.tensor], lambda x, w, out, aux=None: [w.local, out, aux], gather_gemm)
    wrap("gemm_scatter", lambda a, b, a_mn, b_mn, dst: [a, b], lambda a, b, a_mn, b_mn, dst: [dst.peers.tensor], lambda *a, **k: None)
    wrap("scatter_to_stage", lambda src, dst: [src], lambda src, dst: [dst.peers.tensor], lambda *a, **k: None)
    wrap("linear_fwd", lambda x, w, out=None: [x] + ([w] if isinstance(w, torch.Tensor) else []), lambda x, w, out=None: [out])
    wrap("linear_swiglu_fwd", lambda x, w, gu, s: [x] + ([w] if isinstance(w, torch.Tensor) else []), lambda x, w, gu, s: [gu, s])
    wrap("embedding_fwd", lambda tok, table, out=None: [table], lambda tok, table, out=None: [out])
    wrap("cross_entropy_", lambda logits, *a, **k: [logits], lambda logits, *a, loss=None, **k: [logits, loss])
    wrap("sumsq_", lambda x, out: [x], lambda x, out: [out])
    wrap("adamw_", lambda master, m, v, grad, param_lp, *a, **k: [grad], lambda master, m, v, grad, param_lp, *a, **k: [master, m, v, param_lp])
    monkeypatch.setattr(tr.engine.attn, "backward",
                        lambda layer, dout, batch, seq, dqkv: (log.add("attention.backward", [dout], [dqkv]), dqkv.zero_()))
    tokens = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(1))
    for _ in range(3):
        tr.train_step(tokens, tokens)
    names = [o[0] for o in log.ops]
    assert names.count("all_gather") == 3 and names.count("copy_segments") == 3  # only the embedding unit and the norm weights
    assert names.count("gemm_gather") == 3 * (4 * cfg.n_layers + 1)
    assert names.count("gemm_scatter") == 3 * (4 * cfg.n_layers + 1) and names.count("reduce_stage") == 3 * (cfg.n_layers + 1)
    assert _check(log) == []


class _LoggingManager:
    """What `EngineDiLoCo` needs of a manager, with the collectives logged on the stream they are issued on."""

    _use_async_quorum = False

    def __init__(self, log):
        self.log, self.step = log, 0

    def register_state_dict_fn(self, *a, **k):
        pass

    def disallow_state_dict_read(self):
        pass

    def allow_state_dict_read(self):
        pass

    def start_quorum(self, *a, **k):
        pass

    def current_step(self):
        return self.step

    def should_commit(self):
        self.step += 1
        return True

    def allreduce(self, tensor, should_quantize=False, **k):
        from torchft_b200.work import _DummyWork

        self.log.add("allreduce", [tensor], [tensor])
        return _DummyWork(tensor)

    def allreduce_delta(self, out, a, b, should_quantize=False):
        from torchft_b200.work import _DummyWork

        self.log.add("allreduce_delta", [a, b], [out])
        out.copy_(a - b)
        return _DummyWork(out)


@pytest.mark.parametrize("delay", [0, 1])
def test_diloco_exchange_stream_is_ordered(monkeypatch, fake_cuda, delay):
    """Streaming DiLoCo on the engine: the pseudo-gradient exchange runs on a stream of its own, with a delay beside
    the next inner step (whose optimizer rewrites the weights the pseudo-gradient was taken from), the outer step
    back on the training stream, the weight-gradient stream inside every inner step."""
    import torchft_b200.parallel.diloco as D

    cfg, B, S = L.LLAMA_TINY, 2, 16
    log = _Log()
    tr = ShardedLlamaTrainer(cfg, B, S, torch.device("cpu"), logit_chunks=1, seed=3)
    tr.engine.wstream = _Stream()
    tr.engine._w_events, tr.engine._w_last = {}, {}
    mgr = _LoggingManager(log)
    d = D.EngineDiLoCo(tr, mgr, n_fragments=2, sync_every=4, fragment_sync_delay=delay)
    d.stream = _Stream()  # the constructor only creates it on a CUDA device
    _instrument(monkeypatch, log)
    real_sub, real_outer = torch.sub, D.outer_step_

    def sub(a, b, *args, out=None, **k):
        if out is not None:
            log.add("sub", [a, b], [out])
        return real_sub(a, b, *args, out=out, **k)

    def outer(g, m, backup, param, *a, **k):
        log.add("outer_step", [g, m, backup, param], [m, backup, param])
        return real_outer(g, m, backup, param, *a, **k)

    monkeypatch.setattr(torch, "sub", sub)
    monkeypatch.setattr(D, "outer_step_", outer)
    for name, reads, writes in (
        ("linear_fwd", lambda x, w, out=None: [x, w], lambda x, w, out=None: [out]),
        ("linear_swiglu_fwd", lambda x, w, gu, s: [x, w], lambda x, w, gu, s: [gu, s]),
        ("embedding_fwd", lambda tok, table, out=None: [table], lambda tok, table, out=None: [out]),
        ("sumsq_", lambda x, out: [x], lambda x, out: [out]),
        ("adamw_", lambda master, m, v, grad, param_lp, *a, **k: [grad, master], lambda master, m, v, grad, param_lp, *a, **k: [master, m, v, param_lp]),
    ):
        fn = getattr(K, name)
        monkeypatch.setattr(K, name, (lambda fn, name, reads, writes: lambda *a, **k: (log.add(name, reads(*a, **k), writes(*a, **k)), fn(*a, **k))[1])(fn, name, reads, writes))
    monkeypatch.setattr(tr.engine.attn, "backward",
                        lambda layer, dout, batch, seq, dqkv: (log.add("attention.backward", [dout], [dqkv]), dqkv.zero_()))
    tokens = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(1))
    for _ in range(8):  # two synchronisations of each fragment
        d.train_step(tokens, tokens)
    assert d.commits == 4
    names = [o for o in log.ops if o[1] == d.stream.id]
    assert names and all(o[0] in ("allreduce", "allreduce_delta") for o in names)
    assert _check(log) == []
