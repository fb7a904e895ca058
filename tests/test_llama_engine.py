"""The explicit forward/backward engine must match autograd on the same weights."""
import pytest
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
