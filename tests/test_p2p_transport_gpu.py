"""The live-recovery copy kernel on one GPU (the sources are local tensors, so no IPC mapping is needed):
bytes arrive, the per-tensor checksums of the source and of the copy agree, a wrong checksum is reported,
and a copy whose transport was aborted returns at once with ABORTED and an untouched destination."""
from datetime import timedelta

import pytest
import torch

pytestmark = pytest.mark.gpu


def _transport():
    from torchft_b200.checkpointing.p2p_transport import P2PTransport

    return P2PTransport(timeout=timedelta(seconds=5), device=torch.device("cuda", 0))


def test_pull_copies_and_checksums_agree():
    from torchft_b200.checkpointing.p2p_transport import _checksums

    tr = _transport()
    try:
        torch.manual_seed(0)
        srcs = [torch.randn(n, device="cuda") for n in (4, 1000, 3_000_003)] + [torch.randn(5001, device="cuda").bfloat16()]
        dsts = [torch.zeros_like(s) for s in srcs]
        sums = _checksums(srcs, torch.device("cuda", 0))
        assert all(s is not None for s in sums)
        segs = [(s.data_ptr(), d.data_ptr(), s.numel() * s.element_size()) for s, d in zip(srcs, dsts)]
        mismatch = tr._pull(segs, sums, timedelta(seconds=5))
        torch.cuda.synchronize()
        assert int(tr._status.item()) == 0 and mismatch() == []
        for s, d in zip(srcs, dsts):
            assert torch.equal(s, d)
        # a source that changed after its checksum was published is noticed
        wrong = list(sums)
        wrong[2] = (wrong[2] + 1) & 0xFFFFFFFFFFFFFFFF
        mismatch = tr._pull(segs, wrong, timedelta(seconds=5))
        torch.cuda.synchronize()
        assert mismatch() == [2]
    finally:
        tr.shutdown(wait=False)


def test_aborted_pull_returns_with_status_and_moves_nothing():
    tr = _transport()
    try:
        src = torch.ones(1 << 22, device="cuda")
        dst = torch.zeros_like(src)
        tr.abort()
        tr._pull([(src.data_ptr(), dst.data_ptr(), src.numel() * 4)], None, timedelta(seconds=5))
        torch.cuda.synchronize()
        assert int(tr._status.item()) == 2  # aborted
        assert float(dst.sum().item()) == 0.0
        assert torch.ones(4, device="cuda").sum().item() == 4.0
    finally:
        tr.shutdown(wait=False)
