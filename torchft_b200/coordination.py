"""Coordination primitives: the Python face of the C++ control plane.

These classes are what a job needs to talk to (or host) a lighthouse and a manager
server without going through :class:`torchft_b200.manager.Manager`, e.g. to build a
custom launcher or a dashboard.  Same surface as ``torchft.coordination`` in the
reference (torchft/coordination.py:1-37), implemented by the in-tree ``_ftcp`` module.

Args: every constructor and call takes ``datetime.timedelta`` timeouts; a deadline that
passes raises ``TimeoutError``, any other control-plane failure ``RuntimeError``.
"""

from ._ftcp import (  # noqa: F401
    LighthouseClient,
    LighthouseServer,
    ManagerClient,
    ManagerServer,
    Quorum,
    QuorumMember,
    QuorumResult,
    Timestamp,
    lighthouse_main,
)

__all__ = [
    "LighthouseClient",
    "LighthouseServer",
    "ManagerServer",
    "ManagerClient",
    "Quorum",
    "QuorumMember",
    "QuorumResult",
    "Timestamp",
    "lighthouse_main",
]
