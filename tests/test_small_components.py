"""OptimizerWrapper, DistributedSampler, DDP wrappers, ParameterServer, coordination
docstrings, structured loggers, launcher plumbing."""
import json
import logging
import threading
from datetime import timedelta
from unittest.mock import MagicMock, create_autospec

import pytest
import torch
from torch import nn, optim
from torch.distributed.distributed_c10d import ReduceOp

from torchft_b200 import coordination
from torchft_b200.data import DistributedSampler
from torchft_b200.ddp import DistributedDataParallel, PureDistributedDataParallel
from torchft_b200.manager import Manager
from torchft_b200.optim import OptimizerWrapper
from torchft_b200.parameter_server import ParameterServer
from torchft_b200.process_group import ProcessGroup, ProcessGroupGloo
from torchft_b200.work import _DummyWork


def test_optimizer_wrapper_gates_step():
    manager = create_autospec(Manager, instance=True)
    model = nn.Linear(3, 4)
    inner = optim.SGD(model.parameters(), lr=1.0)
    opt = OptimizerWrapper(manager, inner)
    opt.zero_grad()
    assert manager.start_quorum.call_count == 1
    before = model.weight.detach().clone()
    model(torch.ones(2, 3)).sum().backward()
    manager.should_commit.return_value = False
    opt.step()
    assert torch.equal(model.weight, before)
    manager.should_commit.return_value = True
    opt.step()
    assert not torch.equal(model.weight, before)
    assert opt.param_groups is inner.param_groups and opt.state is inner.state
    opt.load_state_dict(opt.state_dict())
    opt.add_param_group({"params": [nn.Parameter(torch.zeros(1))]})
    assert len(inner.param_groups) == 2
    with pytest.raises(AssertionError):
        opt.step(closure=lambda: 0)


def test_distributed_sampler_sharding():
    data = list(range(1000))
    s = DistributedSampler(data, replica_rank=1, num_replica_groups=2, group_rank=3, num_replicas=4, shuffle=False)
    assert s.global_rank == 3 + 4 * 1 and s.global_world_size == 8
    idx = list(iter(s))
    assert idx[0] == 7 and idx[1] == 15 and len(idx) == 125


def _mock_manager():
    m = create_autospec(Manager, instance=True)
    m.allreduce.side_effect = lambda t, should_quantize=False, reduce_op=ReduceOp.AVG: _DummyWork(t)
    return m


def test_ddp_calls_manager_allreduce_per_bucket():
    m = _mock_manager()
    model = nn.Sequential(nn.Linear(3, 4), nn.Linear(4, 2))
    ddp = DistributedDataParallel(m, model)
    ddp(torch.ones(5, 3)).sum().backward()
    assert m.allreduce.call_count >= 1
    assert all(p.grad is not None for p in model.parameters())


def test_pure_ddp_one_allreduce_per_parameter():
    m = _mock_manager()
    model = nn.Sequential(nn.Linear(3, 4), nn.Linear(4, 2))
    ddp = PureDistributedDataParallel(m, model)
    ddp(torch.ones(5, 3)).sum().backward()
    assert m.allreduce.call_count == len(list(model.parameters()))


def test_parameter_server_session():
    class PS(ParameterServer):
        @classmethod
        def new_process_group(cls) -> ProcessGroup:
            return ProcessGroupGloo(timeout=timedelta(seconds=10))

        def forward(self, session_id: str, pg: ProcessGroup) -> None:
            t = torch.zeros(3)
            pg.broadcast_one(t, root=1).wait()       # client -> server
            pg.broadcast_one(t * 2, root=0).wait()   # server -> client
            pg.shutdown()

    ps = PS(port=0)
    try:
        pg = PS.new_session(ps.address())
        x = torch.arange(3.0)
        pg.broadcast_one(x, root=1).wait()
        out = torch.zeros(3)
        pg.broadcast_one(out, root=0).wait()
        assert torch.equal(out, x * 2)
        pg.shutdown()
    finally:
        ps.shutdown()


def test_coordination_api_is_documented():
    for name in coordination.__all__:
        assert hasattr(coordination, name)
    assert "Args:" in coordination.__doc__


def test_structured_loggers_carry_fields():
    from torchft_b200.otel import _FieldFormatter, setup_logger

    lg = setup_logger("torchft_commits")
    records = []

    class H(logging.Handler):
        def emit(self, r):
            records.append(r)

    h = H()
    lg.addHandler(h)
    try:
        lg.info("", extra={"job_id": "j", "replica_id": "r", "rank": 0, "quorum_id": 3, "step": 9, "commit_result": True})
    finally:
        lg.removeHandler(h)
    line = _FieldFormatter().format(records[0])
    assert "quorum_id=3" in line and "commit_result=True" in line and "step=9" in line


def test_runner_environment_and_punisher(tmp_path):
    from torchft_b200.launch.runner import Punisher, Runner

    r = Runner(["train.py"], num_groups=2, gpus_per_group=4, lighthouse_addr="http://x:1", pid_file=str(tmp_path / "p.json"))
    env = r._env(1)
    assert env["REPLICA_GROUP_ID"] == "1" and env["NUM_REPLICA_GROUPS"] == "2" and env["CUDA_VISIBLE_DEVICES"] == "4,5,6,7"
    (tmp_path / "p.json").write_text(json.dumps({"0": None, "1": None}))
    assert Punisher(str(tmp_path / "p.json")).kill_one() is None
