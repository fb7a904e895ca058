"""Type stub of the C++ control-plane extension module (``csrc/control/bindings.cpp``).

Blocking calls release the GIL.  A deadline that passes raises ``TimeoutError``; any other control-plane
failure raises ``RuntimeError``."""

from datetime import timedelta
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

class Timestamp:
    seconds: int
    nanos: int
    def __init__(self) -> None: ...

class QuorumMember:
    replica_id: str
    address: str
    store_address: str
    step: int
    world_size: int
    shrink_only: bool
    data: Optional[Dict[str, object]]
    commit_failures: int
    def __init__(
        self,
        replica_id: str,
        address: str = "",
        store_address: str = "",
        step: int = 0,
        world_size: int = 0,
        shrink_only: bool = False,
        data: Optional[Dict[str, object]] = None,
        commit_failures: int = 0,
    ) -> None: ...

class Quorum:
    quorum_id: int
    participants: List[QuorumMember]
    created: Timestamp
    def __init__(self) -> None: ...

class QuorumResult:
    quorum_id: int
    replica_rank: int
    replica_world_size: int
    recover_src_manager_address: str
    recover_src_replica_rank: Optional[int]
    recover_dst_replica_ranks: List[int]
    store_address: str
    max_step: int
    max_replica_rank: Optional[int]
    max_world_size: int
    heal: bool
    commit_failures: int
    def __init__(self) -> None: ...

class ManagerClient:
    def __init__(self, addr: str, connect_timeout: timedelta) -> None: ...
    def _quorum(
        self,
        group_rank: int,
        step: int,
        checkpoint_metadata: str,
        shrink_only: bool,
        timeout: timedelta,
        init_sync: bool = True,
        commit_failures: int = 0,
    ) -> QuorumResult: ...
    def _checkpoint_metadata(self, rank: int, timeout: timedelta) -> str: ...
    def should_commit(self, group_rank: int, step: int, should_commit: bool, timeout: timedelta) -> bool: ...
    def _kill(self, msg: str, timeout: timedelta) -> None: ...

class ManagerServer:
    def __init__(
        self,
        replica_id: str,
        lighthouse_addr: str,
        hostname: str,
        bind: str,
        store_addr: str,
        world_size: int,
        heartbeat_interval: timedelta,
        connect_timeout: timedelta,
        quorum_retries: int = 0,
    ) -> None: ...
    def address(self) -> str: ...
    def shutdown(self) -> None: ...

class LighthouseServer:
    def __init__(
        self,
        bind: str,
        min_replicas: int,
        join_timeout_ms: Optional[int] = None,
        quorum_tick_ms: Optional[int] = None,
        heartbeat_timeout_ms: Optional[int] = None,
    ) -> None: ...
    def address(self) -> str: ...
    def shutdown(self) -> None: ...

class LighthouseClient:
    def __init__(self, addr: str, connect_timeout: timedelta) -> None: ...
    def quorum(
        self,
        replica_id: str,
        timeout: timedelta,
        address: Optional[str] = None,
        store_address: Optional[str] = None,
        step: Optional[int] = None,
        world_size: Optional[int] = None,
        shrink_only: Optional[bool] = None,
        data: Optional[Dict[str, object]] = None,
    ) -> Quorum: ...
    def heartbeat(self, replica_id: str, timeout: timedelta = ...) -> None: ...

def lighthouse_main(argv: Optional[Sequence[str]] = None) -> int: ...

# The quorum mathematics as pure functions (used by the table-driven tests).  Times are seconds on an arbitrary clock.
def quorum_compute(
    now: float,
    participants: Sequence[Tuple[QuorumMember, float]],
    heartbeats: Mapping[str, float],
    prev_quorum: Optional[Quorum] = None,
    min_replicas: int = 1,
    join_timeout_ms: int = 60000,
    heartbeat_timeout_ms: int = 5000,
) -> Tuple[Optional[List[QuorumMember]], str]: ...
def compute_quorum_results(replica_id: str, group_rank: int, quorum: Quorum, init_sync: bool = True) -> QuorumResult: ...
def quorum_changed(a: Sequence[QuorumMember], b: Sequence[QuorumMember]) -> bool: ...
