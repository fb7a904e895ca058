"""The explicit forward/backward engine must match autograd on the same weights."""
import torch

from torchft_b200.models.llama import LLAMA_TINY, TorchLlama
from torchft_b200.parallel.hsdp import ShardedLlamaTrainer


def _oracle(trainer, cfg, tokens, targets, dtype):
    ref = TorchLlama(cfg).to(tokens.device, dtype)
    ref.load_units(lambda u: trainer._param_unit(u))
    logits = ref(tokens).float()
    loss = torch.nn.functional.cross_entropy(logits.view(-1, cfg.vocab_size), targets.view(-1))
    loss.backward()
    return ref, loss


def test_engine_matches_autograd_cpu():
    torch.manual_seed(0)
    cfg = LLAMA_TINY
    B, S = 2, 16
    dev = torch.device("cpu")
    tr = ShardedLlamaTrainer(cfg, B, S, dev, logit_chunks=2)
    tokens = torch.randint(0, cfg.vocab_size, (B, S))
    targets = torch.randint(0, cfg.vocab_size, (B, S))
    loss = tr.forward_backward(tokens, targets)
    ref, ref_loss = _oracle(tr, cfg, tokens, targets, torch.float32)
    assert abs(loss.item() - ref_loss.item()) < 3e-2
    from torchft_b200.models.llama import _Fields

    g = _Fields(tr._grad_unit(1), cfg.unit_fields(1))
    for name in ("wqkv", "wo", "wgu", "wd", "attn_norm", "ffn_norm"):
        got = getattr(g, name).float()
        want = getattr(ref.layers[0], name).grad
        err = (got - want).norm() / (want.norm() + 1e-12)
        assert err < 0.08, (name, err.item())
    ge = _Fields(tr._grad_unit(0), cfg.unit_fields(0)).tok_embeddings.float()
    err = (ge - ref.tok_embeddings.grad).norm() / ref.tok_embeddings.grad.norm()
    assert err < 0.08
    tr.optimizer_step()
    l2 = tr.forward_backward(tokens, targets)
    assert l2.item() < loss.item()


def test_kept_norm_outputs_give_the_same_gradients_as_recomputed_ones():
    """`save_norms`: the forward pass keeps the normalised GEMM inputs per layer instead of recomputing them in the
    backward pass; same kernels on the same values, so the gradients are bit-identical."""
    cfg, B, S = LLAMA_TINY, 2, 16
    dev = torch.device("cpu")
    tokens = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(5))
    targets = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(6))
    grads = []
    for keep in (False, True):
        tr = ShardedLlamaTrainer(cfg, B, S, dev, logit_chunks=1, seed=11, save_norms=keep)
        assert (tr.engine.n1 is not None) == keep
        tr.forward_backward(tokens, targets)
        grads.append([tr._grad_unit(u).clone() for u in range(cfg.n_units)])
    for a, b in zip(*grads):
        assert torch.equal(a, b)


def test_sharded_trainer_two_gloo_ranks(tmp_path):
    """Two CPU ranks, parameters, gradients and optimizer state sharded between them, each with its own
    micro-batch: the reduce-scattered gradient equals the gradient one process computes on both
    micro-batches at once (the shard group's gradient is the mean over all of its tokens), and training
    on the shards makes progress."""
    import json
    import os
    import socket
    import subprocess
    import sys

    cfg, S = LLAMA_TINY, 16
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_hsdp_cpu_worker.py")
    out_path = str(tmp_path / "grads.pt")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(port), out_path], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(2)]
    res = []
    for p in procs:
        out, err = p.communicate(timeout=300)
        assert p.returncode == 0, err[-3000:]
        res.append(json.loads([l for l in out.splitlines() if l.startswith("{")][-1]))
    res.sort(key=lambda r: r["rank"])
    grads = torch.load(out_path)

    g = torch.Generator().manual_seed(7)
    tok = torch.randint(0, cfg.vocab_size, (2, S + 1), generator=g)
    ref = ShardedLlamaTrainer(cfg, 2, S, torch.device("cpu"), seed=3, lr=1e-2, max_grad_norm=1e9)
    ref_loss = float(ref.forward_backward(tok[:, :-1], tok[:, 1:]))
    assert abs(ref_loss - 0.5 * (res[0]["losses"][0] + res[1]["losses"][0])) < 2e-2
    for u in range(cfg.n_units):
        want = ref.g_shard[u][: cfg.unit_numel(u)].float()
        err = (grads[u] - want).norm() / (want.norm() + 1e-12)
        assert err < 3e-2, (u, float(err))
    for r in res:  # the same micro-batch every step: the loss has to fall
        assert r["losses"][-1] < r["losses"][0]


def test_shard_pieces_cut_a_field_at_shard_boundaries():
    """The fused all-gather copies small fields (norm weights) piecewise from their owners."""
    from torchft_b200.parallel.hsdp import shard_pieces

    assert shard_pieces(10, 30, 16) == [(0, 10, 10, 6), (1, 0, 16, 16), (2, 0, 32, 8)]
    assert shard_pieces(0, 8, 8) == [(0, 0, 0, 8)]
    assert shard_pieces(16, 16, 16) == [(1, 0, 16, 16)]
    for off, n, shard in ((5, 3, 100), (96, 4096, 1000), (0, 1, 1)):
        pieces = shard_pieces(off, n, shard)
        assert sum(p[3] for p in pieces) == n
        assert pieces[0][2] == off and all(a[2] + a[3] == b[2] for a, b in zip(pieces, pieces[1:]))
        assert all(o * shard + s == u and s + c <= shard for o, s, u, c in pieces)
