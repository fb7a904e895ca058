"""ProcessGroupB200 on one GPU: the whole c10d surface on a group of one (shapes, dtypes, works), and
the rule that a failed shard-group kernel turns the step's commit vote into a no."""
import ctypes
from datetime import timedelta
from unittest.mock import MagicMock

import pytest
import torch
import torch.distributed as dist
from torch.distributed.distributed_c10d import (AllgatherOptions, AllreduceOptions, AllToAllOptions, BarrierOptions,
                                                BroadcastOptions, ReduceScatterOptions)

pytestmark = pytest.mark.gpu


def test_world_of_one_runs_every_collective():
    from torchft_b200.parallel.team import ProcessGroupB200

    store = dist.TCPStore("localhost", 0, is_master=True, wait_for_workers=False)
    pg = ProcessGroupB200(timeout=timedelta(seconds=5), arena_bytes=1 << 20, staging_bytes=1 << 20, p2p_bytes=1 << 20)
    pg.configure(f"localhost:{store.port}/torchft/1/0", "r", 0, 1)
    t = torch.arange(6, dtype=torch.float32, device="cuda").reshape(2, 3)
    for dtype in (torch.float32, torch.bfloat16, torch.int64):
        x = t.to(dtype)
        out = torch.empty_like(x)
        pg.allgather([[out]], [x], AllgatherOptions()).wait()
        assert torch.equal(out, x)
        out.zero_()
        pg.allgather_into_tensor_coalesced([out], [x], AllgatherOptions()).wait()
        assert torch.equal(out, x)
        out.zero_()
        pg.alltoall_base(out, x, [], [], AllToAllOptions()).wait()
        assert torch.equal(out, x)
        y = x.clone()
        pg.broadcast([y], BroadcastOptions()).wait()
        pg.broadcast_one(y, 0).wait()
        assert torch.equal(y, x)
    for dtype in (torch.float32, torch.bfloat16):
        x = t.to(dtype)
        y = x.clone()
        w = pg.allreduce([y], AllreduceOptions())
        w.wait()
        w.get_future().wait()
        pg.allreduce_coalesced([y, y.clone()]).wait()
        assert torch.equal(y, x)
        out = torch.empty_like(x)
        pg.reduce_scatter([out], [[x]], ReduceScatterOptions()).wait()
        assert torch.equal(out, x)
        out.zero_()
        pg.reduce_scatter_tensor_coalesced([out], [x], ReduceScatterOptions()).wait()
        assert torch.equal(out, x)
    pg.barrier(BarrierOptions()).wait()
    assert pg.errored() is None and pg.size() == 1
    with pytest.raises(NotImplementedError):
        pg.alltoall_base(torch.empty(4, device="cuda"), torch.empty(4, device="cuda"), [1, 3], [1, 3])
    pg.shutdown()


def test_failed_shard_team_kernel_declines_the_commit():
    """A shard-group kernel whose peer never arrives returns with TIMEOUT in the team's status word and stale data
    behind it.  The trainer must read that word before the vote: the manager gets the error (its vote is then no)
    and the optimizer does not run."""
    from torchft_b200.models.llama import LlamaConfig
    from torchft_b200.parallel.hsdp import ShardedLlamaTrainer
    from torchft_b200.parallel.team import SymmetricTeam, TeamError

    dev = torch.device("cuda", 0)
    team = SymmetricTeam(dev, 1 << 20, timeout=timedelta(seconds=0.2))
    # a world of two whose second member is only memory: nothing ever signals from there
    ghost = torch.zeros(1 << 20, dtype=torch.uint8, device=dev)
    team.rank, team.world, team.epoch = 0, 2, 5
    team.peer_base = [team.arena.base, ghost.data_ptr()]
    off = team.arena.alloc(2 * 8 * 64 * 2)
    team.allreduce_(off, 2 * 8 * 64, torch.bfloat16)
    torch.cuda.synchronize()
    assert team.status() == 1

    cfg = LlamaConfig(dim=256, n_layers=1, n_heads=2, n_kv_heads=1, ffn_dim=512, vocab_size=512, name="tiny")
    manager = MagicMock()
    errors = []
    manager.report_error.side_effect = errors.append
    manager.should_commit.side_effect = lambda: not errors
    manager.allreduce.side_effect = lambda t, **kw: MagicMock()
    tr = ShardedLlamaTrainer(cfg, 1, 128, dev, manager=manager, logit_chunks=1)
    tr.comm.team = team  # what PeerShardComm exposes
    tok = torch.randint(0, cfg.vocab_size, (1, 129), device=dev)
    tr.train_step(tok[:, :-1], tok[:, 1:])
    assert len(errors) == 1 and isinstance(errors[0], TeamError) and "timeout" in str(errors[0])
    assert tr.opt_step == 0
    # without a manager the failure is raised
    tr.manager = None
    with pytest.raises(TeamError):
        tr.train_step(tok[:, :-1], tok[:, 1:])
