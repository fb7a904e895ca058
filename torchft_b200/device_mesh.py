"""Device-mesh glue for HSDP: a mesh whose replicate dimension is fault tolerant.

``torch.distributed.DeviceMesh`` assumes fixed world sizes.  :func:`ft_init_device_mesh`
builds the real mesh over the dimensions *inside* a replica group (shard, tensor, ...)
and wraps it in a :class:`ManagedDeviceMesh` that answers every DeviceMesh query as if a
replicate dimension of size ``manager.num_participants()`` existed in addition; the
group of that dimension is a :class:`~torchft_b200.process_group.ManagedProcessGroup`,
so FSDP2's replicate-dimension allreduce becomes ``Manager.allreduce``.
Counterpart of torchft/device_mesh.py:22-340.
"""

from __future__ import annotations

import warnings
from typing import TYPE_CHECKING, Any, Dict, List, Optional, Tuple, Union

import torch
from torch.distributed import ProcessGroup as BaseProcessGroup
from torch.distributed import get_rank
from torch.distributed.device_mesh import DeviceMesh, _mesh_resources, init_device_mesh

from .process_group import ManagedProcessGroup, ProcessGroup

if TYPE_CHECKING:
    from .manager import Manager


def extend_device_mesh(mesh: DeviceMesh, pg: ProcessGroup, name: str = "dp", dim: int = 0) -> DeviceMesh:
    """Older helper: insert ``pg`` into ``mesh`` as a new dimension ``name`` of size 1.
    DeviceMesh believes the dimension has one member; the scaling by the real number of
    replicas happens inside ``pg``.  ``pg`` must have been registered (``pg.register(name)``) so that torch can
    resolve it by name."""
    try:
        pg.group_name
    except ValueError as e:
        raise ValueError("extend_device_mesh needs a registered process group: call pg.register(<name>) first") from e
    groups = mesh.get_all_groups()
    groups.insert(dim, pg)
    names = list(mesh.mesh_dim_names or [])
    names.insert(dim, name)
    return DeviceMesh.from_group(group=groups, device_type=mesh.device_type, mesh=mesh.mesh.unsqueeze(dim),
                                 mesh_dim_names=tuple(names))


class ManagedDeviceMesh(DeviceMesh):
    """DeviceMesh facade: ``mesh`` covers the real dimensions, ``replicate_pg`` stands in
    for dimension ``replicate_dim``.  Instances are picklable: the process group is
    re-attached from a per-process singleton on unpickling."""

    replicate_pg_singleton: Optional[ManagedProcessGroup] = None

    def __init__(self, mesh: Optional[DeviceMesh], mesh_dim_names: Tuple[str, ...], replicate_pg: ManagedProcessGroup,
                 replicate_dim: int, parent: Optional["ManagedDeviceMesh"]) -> None:
        if mesh is None and parent is None:
            raise ValueError("ManagedDeviceMesh doesn't support both mesh and parent are None.")
        self._mesh = mesh
        self._mesh_dim_names = tuple(mesh_dim_names)
        self.replicate_pg = replicate_pg
        self.replicate_dim = replicate_dim
        self.replicate_dim_name: str = mesh_dim_names[replicate_dim]
        self.parent = parent
        self.flatten_meshes: Dict[str, DeviceMesh] = {}
        src = mesh if mesh is not None else parent
        assert src is not None
        self._device_type: str = src.device_type
        self._flatten_mesh_list: Tuple[DeviceMesh, ...] = tuple()
        self._flatten_mapping: Dict[str, DeviceMesh] = {}
        self._thread_id: Optional[int] = None
        self._hash: Optional[int] = None

    # ---- pickling
    def __getstate__(self) -> Dict[str, Any]:
        state = self.__dict__.copy()
        state["replicate_pg"] = None
        return state

    def __setstate__(self, state: Dict[str, Any]) -> None:
        self.__dict__.update(state)
        assert self.replicate_pg_singleton is not None
        self.replicate_pg = self.replicate_pg_singleton

    # ---- slicing
    def __getitem__(self, mesh_dim_names: Union[str, Tuple[str, ...]]) -> DeviceMesh:
        if isinstance(mesh_dim_names, str):
            if mesh_dim_names == self.replicate_dim_name:
                sub: DeviceMesh = ManagedDeviceMesh(None, (mesh_dim_names,), self.replicate_pg, 0, parent=self)
            elif mesh_dim_names in self.flatten_meshes:
                sub = self.flatten_meshes[mesh_dim_names]
            else:
                assert self._mesh is not None
                sub = self._mesh[mesh_dim_names]
        else:
            assert isinstance(mesh_dim_names, tuple)
            if self.replicate_dim_name not in mesh_dim_names:
                assert self._mesh is not None
                sub = self._mesh[mesh_dim_names]
            else:
                rest = tuple(n for n in mesh_dim_names if n != self.replicate_dim_name)
                assert self._mesh is not None
                sub = ManagedDeviceMesh(self._mesh[rest], mesh_dim_names, self.replicate_pg,
                                        mesh_dim_names.index(self.replicate_dim_name), parent=self)
        try:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")  # torch announces the removal of this lookup; there is no public successor yet
                sub._root_mesh = _mesh_resources.get_root_mesh(self)  # type: ignore[attr-defined]
        except Exception:
            pass
        return sub

    def _real_mesh_dim(self, mesh_dim: int) -> int:
        return mesh_dim - 1 if mesh_dim > self.replicate_dim else mesh_dim

    def _dim_index(self, mesh_dim: Optional[Union[int, str]]) -> int:
        if isinstance(mesh_dim, str):
            return self._mesh_dim_names.index(mesh_dim)
        return 0 if mesh_dim is None else int(mesh_dim)

    # ---- queries
    @property
    def mesh_dim_names(self) -> Tuple[str, ...]:  # type: ignore[override]
        return self._mesh_dim_names

    @property
    def device_type(self) -> str:  # type: ignore[override]
        return self._device_type

    def get_group(self, mesh_dim: Optional[Union[int, str]] = None) -> BaseProcessGroup:
        dim = self._dim_index(mesh_dim)
        if mesh_dim is None or dim == self.replicate_dim:
            return self.replicate_pg
        assert self._mesh is not None
        return self._mesh.get_group(self._real_mesh_dim(dim))

    def _flatten(self, mesh_dim_name: Optional[str] = None, backend_override=None) -> DeviceMesh:
        if mesh_dim_name is None:
            raise ValueError("ManagedDeviceMesh._flatten requires `mesh_dim_name`")
        flat = _FlattenDeviceMesh(self)
        (self if self.parent is None else self.parent).flatten_meshes[mesh_dim_name] = flat
        return flat

    def size(self, mesh_dim: Optional[int] = None) -> int:
        # before the first quorum the manager reports 0 participants; present that as 1
        rep = self.replicate_pg.size() or 1
        if mesh_dim is None:
            return rep if self._mesh is None else self._mesh.size() * rep
        if mesh_dim == self.replicate_dim:
            return rep
        assert self._mesh is not None
        return self._mesh.size(self._real_mesh_dim(mesh_dim))

    @property
    def ndim(self) -> int:
        assert self._mesh is not None
        return self._mesh.ndim + 1

    @property
    def shape(self) -> Tuple[int, ...]:
        assert self._mesh is not None
        dims = list(self._mesh.shape)
        dims.insert(self.replicate_dim, self.replicate_pg.size())
        return tuple(dims)

    def get_rank(self) -> int:
        assert self._mesh is not None
        return self._mesh.get_rank()

    def get_local_rank(self, mesh_dim: Optional[Union[int, str]] = None) -> int:
        dim = self._dim_index(mesh_dim)
        if mesh_dim is None:
            if self._mesh is None:
                return get_rank(self.replicate_pg)
            assert self.replicate_dim == 0, "replicate_dim must be the first one"
            return self._mesh.size() * get_rank(self.replicate_pg) + self._mesh.get_local_rank()
        if dim == self.replicate_dim:
            return get_rank(self.replicate_pg)
        assert self._mesh is not None
        return self._mesh.get_local_rank(self._real_mesh_dim(dim))

    def get_coordinate(self) -> Optional[List[int]]:
        """This rank's index along every dimension, the replicate dimension included."""
        assert self._mesh is not None
        coord = self._mesh.get_coordinate()
        if not coord:
            return coord
        coord = list(coord)
        coord.insert(self.replicate_dim, get_rank(self.replicate_pg))
        return coord

    # DTensor's redistribution code (full_tensor(), state-dict gathering) asks the mesh these two questions through
    # private members of torch's DeviceMesh; answer them from the managed view.
    @property
    def _coordinate_on_dim(self) -> Optional[List[int]]:  # type: ignore[override]
        return self.get_coordinate()

    def _is_current_rank_part_of_mesh(self) -> bool:
        return self.get_coordinate() is not None

    @property
    def _dim_group_names(self) -> List[str]:  # type: ignore[override]
        """Registered group name per mesh dimension: the real mesh's names with the managed group's name inserted at
        the replicate dimension (functional collectives resolve ``(mesh, dim)`` through this list)."""
        names = list(self._mesh._dim_group_names) if self._mesh is not None else []
        names.insert(self.replicate_dim, self.replicate_pg.group_name)
        return names

    # FSDP2 on parameters that are already tensor-parallel DTensors concatenates the data-parallel mesh (this object)
    # with the tensor-parallel mesh (torch's ``DeviceMesh._concatenate``), which reads the members below.  The managed
    # dimension is described as a dimension of size one: its real size lives in the quorum, no rank layout exists for
    # it, and the only collective FSDP runs over it (the gradient all-reduce) goes through ``get_group``, not through
    # the concatenated mesh.
    @property
    def _layout(self):  # type: ignore[override]
        from torch.distributed._mesh_layout import _MeshLayout

        if self._mesh is None:  # the replicate dimension on its own
            return _MeshLayout((1,), (0,))
        real = self._mesh._layout
        sizes = [real[i].sizes for i in range(len(real))]
        strides = [real[i].strides for i in range(len(real))]
        sizes.insert(self.replicate_dim, 1)
        strides.insert(self.replicate_dim, 0)
        return _MeshLayout(tuple(sizes), tuple(strides))

    def _real_source(self) -> DeviceMesh:
        src = self._mesh if self._mesh is not None else (self.parent._mesh if self.parent is not None else None)
        assert src is not None
        return src

    @property
    def _flatten_rank_map(self):  # type: ignore[override]
        return self._real_source()._flatten_rank_map

    @property
    def _rank_map(self):  # type: ignore[override]
        return self._real_source()._rank_map

    def _get_root_mesh(self) -> DeviceMesh:
        return self._real_source()._get_root_mesh()

    def get_all_groups(self) -> List[BaseProcessGroup]:
        """One process group per dimension: the real mesh's groups with the managed group at the replicate dimension."""
        groups: List[BaseProcessGroup] = list(self._mesh.get_all_groups()) if self._mesh is not None else []
        groups.insert(self.replicate_dim, self.replicate_pg)
        return groups

    def __repr__(self) -> str:
        return f"ManagedDeviceMesh(mesh={self._mesh})"

    def __hash__(self) -> int:
        if not self._hash:
            self._hash = hash((self._mesh, self._mesh_dim_names, id(self.replicate_pg), self.replicate_dim,
                               self.replicate_dim_name, self.parent, self._device_type))
        return self._hash

    def __eq__(self, other: object) -> bool:
        return self is other or (isinstance(other, ManagedDeviceMesh) and hash(self) == hash(other))


class _FlattenDeviceMesh(DeviceMesh):
    """What ``ManagedDeviceMesh._flatten`` returns: only size and local rank are meaningful."""

    def __init__(self, managed_mesh: ManagedDeviceMesh) -> None:
        self.managed_mesh = managed_mesh

    def __getitem__(self, mesh_dim_names):
        raise NotImplementedError

    def get_group(self, mesh_dim=None) -> BaseProcessGroup:
        raise NotImplementedError

    def _flatten(self, mesh_dim_name=None, backend_override=None) -> DeviceMesh:
        raise NotImplementedError

    def size(self, mesh_dim: Optional[int] = None) -> int:
        assert mesh_dim is None
        return self.managed_mesh.size()

    @property
    def ndim(self) -> int:
        raise NotImplementedError

    @property
    def shape(self) -> Tuple[int, ...]:
        raise NotImplementedError

    def get_rank(self) -> int:
        raise NotImplementedError

    def get_local_rank(self, mesh_dim=None) -> int:
        assert mesh_dim is None
        return self.managed_mesh.get_local_rank()

    def get_all_groups(self) -> List[BaseProcessGroup]:
        raise NotImplementedError

    def __hash__(self) -> int:
        return hash(("flatten", self.managed_mesh))

    def __repr__(self) -> str:
        return f"_FlattenDeviceMesh({self.managed_mesh})"


def ft_init_device_mesh(*, device_type: str, mesh_shape: Union[Tuple[int, ...], List[int]],
                        mesh_dim_names: Union[Tuple[str, ...], List[str]], replicate_dim: int,
                        manager: "Manager") -> ManagedDeviceMesh:
    """Build an HSDP mesh.  ``mesh_shape[replicate_dim]`` is ignored (the replicate size is
    whatever the quorum says); the remaining dimensions are initialised with
    ``init_device_mesh`` over the ranks of this replica group."""
    shape = list(mesh_shape)
    shape.pop(replicate_dim)
    names = list(mesh_dim_names)
    names.pop(replicate_dim)
    mesh = init_device_mesh(device_type, mesh_shape=tuple(shape), mesh_dim_names=tuple(names))
    replicate_pg = ManagedProcessGroup(manager)
    replicate_pg.register(mesh_dim_names[replicate_dim])
    ManagedDeviceMesh.replicate_pg_singleton = replicate_pg
    return ManagedDeviceMesh(mesh=mesh, mesh_dim_names=tuple(mesh_dim_names), replicate_pg=replicate_pg,
                             replicate_dim=replicate_dim, parent=None)
