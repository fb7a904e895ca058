"""ManagedDeviceMesh over real gloo ranks (spawned processes): the replicate dimension is
answered by the manager, the other dimensions by a real DeviceMesh."""
import os
import pickle
from unittest.mock import MagicMock

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from conftest import free_port


def _worker(rank: int, world: int, port: int) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torchft_b200.device_mesh import ManagedDeviceMesh, ft_init_device_mesh
        from torchft_b200.manager import Manager
        from torchft_b200.process_group import ProcessGroupGloo

        manager = MagicMock(spec=Manager)
        manager._pg = ProcessGroupGloo()
        manager.num_participants.return_value = 0
        mesh = ft_init_device_mesh(device_type="cpu", mesh_shape=(2, world), mesh_dim_names=("dp_replicate", "dp_shard"),
                                   replicate_dim=0, manager=manager)
        assert mesh.ndim == 2
        assert mesh.size(1) == world and mesh.get_local_rank("dp_shard") == rank
        assert mesh["dp_shard"].size() == world
        for n in (0, 1, 2):  # before any quorum the replicate size reads as 1
            manager.num_participants.return_value = n
            assert mesh.size() == world * max(n, 1)
            assert mesh.size(0) == max(n, 1)
        manager.num_participants.return_value = 2
        assert mesh.shape == (2, world)
        rep = mesh["dp_replicate"]
        assert isinstance(rep, ManagedDeviceMesh) and rep.size() == 2
        assert mesh.get_group("dp_replicate") is mesh.replicate_pg
        groups = mesh.get_all_groups()
        assert len(groups) == 2 and groups[0] is mesh.replicate_pg and groups[1] is mesh.get_group("dp_shard")
        both = mesh[("dp_replicate", "dp_shard")]
        assert both.size() == 2 * world
        flat = mesh._flatten("dp")
        assert flat.size() == 2 * world
        assert mesh["dp"] is flat
        coord = mesh.get_coordinate()
        assert coord is not None and len(coord) == 2 and coord[1] == rank
        clone = pickle.loads(pickle.dumps(mesh))
        assert clone.replicate_pg is mesh.replicate_pg
        assert hash(mesh) == hash(mesh) and "ManagedDeviceMesh" in repr(mesh)
    finally:
        dist.destroy_process_group()


def test_managed_device_mesh_gloo():
    world = 2
    port = free_port()
    mp.spawn(_worker, args=(world, port), nprocs=world, join=True)


def _fsdp_worker(rank: int, world: int, port: int, ckpt_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch.distributed.fsdp import fully_shard

        from torchft_b200.device_mesh import ft_init_device_mesh
        from torchft_b200.manager import Manager
        from torchft_b200.process_group import ProcessGroupGloo
        from torchft_b200.work import _DummyWork

        manager = MagicMock(spec=Manager)
        manager._pg = ProcessGroupGloo()
        manager.num_participants.return_value = 1
        seen = []

        def allreduce(t, should_quantize=False, reduce_op=None):
            seen.append(t.numel())
            return _DummyWork(t)

        manager.allreduce.side_effect = allreduce
        mesh = ft_init_device_mesh(device_type="cpu", mesh_shape=(1, world), mesh_dim_names=("dp_replicate", "dp_shard"),
                                   replicate_dim=0, manager=manager)
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
        ref = pickle.loads(pickle.dumps(model))
        fully_shard(model, mesh=mesh)
        # gathering works on the managed mesh too: DTensor.full_tensor() and torch's full state dict
        from torch.distributed.checkpoint.state_dict import StateDictOptions, get_model_state_dict

        for p, q in zip(model.parameters(), ref.parameters()):
            torch.testing.assert_close(p.full_tensor(), q.detach())
        full_sd = get_model_state_dict(model, options=StateDictOptions(full_state_dict=True))
        for k, v in ref.state_dict().items():
            torch.testing.assert_close(full_sd[k], v)
        # ... and so does torch.distributed.checkpoint: sharded save, wipe, sharded load
        import torch.distributed.checkpoint as dcp

        dcp.save({"model": model.state_dict()}, checkpoint_id=ckpt_dir)
        with torch.no_grad():
            for p in model.parameters():
                p.to_local().zero_()
        dcp.load({"model": model.state_dict()}, checkpoint_id=ckpt_dir)
        for p, q in zip(model.parameters(), ref.parameters()):
            torch.testing.assert_close(p.full_tensor(), q.detach())
        x = torch.randn(4 * world, 8)  # the same global batch everywhere; each rank takes its rows
        mine = x[rank * 4:(rank + 1) * 4]
        model(mine).sum().backward()
        ref(x).sum().backward()
        # the shard-sized gradients went through the manager (the replicate dimension) exactly once
        assert len(seen) == 1 and seen[0] > 0
        for p, q in zip(model.parameters(), ref.parameters()):
            # FSDP shards dim 0 over the group and averages over it: this rank holds its rows of the mean gradient
            want = (q.grad / world).chunk(world, dim=0)[rank]
            torch.testing.assert_close(p.grad.to_local(), want, rtol=1e-5, atol=1e-6)
    finally:
        dist.destroy_process_group()


def test_fully_shard_on_managed_mesh_gloo(tmp_path):
    """HSDP as the reference wires it (torchft/fsdp_test.py:82-92): FSDP2 shards inside the group over a real
    process group and reduces over the replicate dimension through the manager."""
    world = 2
    port = free_port()
    mp.spawn(_fsdp_worker, args=(world, port, str(tmp_path / "dcp")), nprocs=world, join=True)


def _tp_worker(rank: int, world: int, port: int) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

        from torchft_b200.device_mesh import ft_init_device_mesh
        from torchft_b200.manager import Manager
        from torchft_b200.process_group import ProcessGroupGloo

        manager = MagicMock(spec=Manager)
        manager._pg = ProcessGroupGloo()
        manager.num_participants.return_value = 1
        mesh = ft_init_device_mesh(device_type="cpu", mesh_shape=(1, 2, 2), mesh_dim_names=("dp_replicate", "dp_shard", "tp"),
                                   replicate_dim=0, manager=manager)
        assert mesh.shape == (1, 2, 2) and mesh["tp"].size() == 2
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 16, bias=False), torch.nn.ReLU(), torch.nn.Linear(16, 8, bias=False))
        w0, w1 = [p.detach().clone() for p in model.parameters()]
        x = torch.randn(4, 8)
        want = torch.relu(x @ w0.t()) @ w1.t()
        parallelize_module(model, mesh["tp"], {"0": ColwiseParallel(), "2": RowwiseParallel()})
        torch.testing.assert_close(model(x), want, rtol=1e-5, atol=1e-5)
        # FSDP2 on top of the tensor-parallel parameters, over the managed (replicate, shard) part of the mesh
        from torch.distributed.fsdp import fully_shard

        from torchft_b200.work import _DummyWork

        seen = []
        manager.allreduce.side_effect = lambda t, should_quantize=False, reduce_op=None: seen.append(t.numel()) or _DummyWork(t)
        fully_shard(model, mesh=mesh["dp_replicate", "dp_shard"])
        out = model(x)
        torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-5)
        out.sum().backward()
        assert len(seen) == 1  # the replicate-dimension reduction of the (shard x tp)-sized gradients went through the manager
        assert all(p.grad is not None for p in model.parameters())
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_and_fsdp2_on_a_3d_managed_mesh():
    """A 3-D managed mesh (replicate x shard x tp): the tp dimension is a real sub-mesh on which torch's tensor-parallel
    styles work, and FSDP2 composes with them over the managed (replicate, shard) part
    (the reference's fsdp_test.py:84-92 builds the same (1, 2, 2) layout)."""
    world = 4
    port = free_port()
    mp.spawn(_tp_worker, args=(world, port), nprocs=world, join=True)


def test_extend_device_mesh_inserts_a_registered_group():
    """The older helper: a registered reconfigurable group becomes an extra mesh dimension of size one; an unregistered
    group is refused with a message that says what to do (torchft/process_group_test.py test_device_mesh).  Child
    process: it initialises torch.distributed."""
    import subprocess
    import sys

    child = r'''
import os, sys
import torch, torch.distributed as dist
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="@PORT@", RANK="0", WORLD_SIZE="1")
dist.init_process_group("gloo", rank=0, world_size=1)
from torch.distributed.device_mesh import init_device_mesh
from torchft_b200.device_mesh import extend_device_mesh
from torchft_b200.process_group import ProcessGroupGloo
store = dist.TCPStore("127.0.0.1", 0, is_master=True, wait_for_workers=False)
pg = ProcessGroupGloo(); pg.configure(f"127.0.0.1:{store.port}/x", "r", 0, 1)
mesh = init_device_mesh("cpu", (1,), mesh_dim_names=("fsdp",))
try:
    extend_device_mesh(mesh, pg); raise SystemExit("expected an error")
except ValueError as e:
    assert "register" in str(e)
pg.register("ext_probe")
ext = extend_device_mesh(mesh, pg)
assert ext.mesh_dim_names == ("dp", "fsdp") and tuple(ext.mesh.shape) == (1, 1), (ext.mesh_dim_names, ext.mesh.shape)
assert ext.get_group("dp").size() == 1
t = torch.ones(3)
dist.all_reduce(t, group=ext.get_group("dp"))
assert torch.equal(t, torch.ones(3))
pg.unregister()
print("extend ok")
'''
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", child.replace("@PORT@", str(free_port()))], capture_output=True, text=True,
                       timeout=240, env=dict(os.environ, PYTHONPATH=repo))
    assert r.returncode == 0 and "extend ok" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
