"""Coordination primitives: the Python face of the C++ control plane.

These classes are what a job needs to talk to (or host) a lighthouse and a manager server without going through
:class:`torchft_b200.manager.Manager`, e.g. to build a custom launcher or a dashboard.  The names and call
signatures are those of ``torchft.coordination`` in the reference (torchft/coordination.py:1-37); the implementation
is the in-tree ``_ftcp`` extension module.

Args: every constructor and call takes ``datetime.timedelta`` timeouts; a deadline that passes raises
``TimeoutError``, any other control-plane failure ``RuntimeError``.  Blocking calls release the GIL.

=====================  ==========================================================================================
``LighthouseServer``   the job-wide quorum service with dashboard (``/``), status (``/status``) and ``/metrics``
``LighthouseClient``   ``quorum(...)`` and ``heartbeat(...)`` against a lighthouse, without a manager
``ManagerServer``      per-replica-group server: gathers the ranks' requests, commit barrier, checkpoint metadata
``ManagerClient``      one per rank: ``_quorum``, ``_checkpoint_metadata``, ``should_commit``
``QuorumResult``       what a rank learns from a quorum round (ranks, recovery assignment, store address)
``Quorum``             a quorum as issued by the lighthouse: id, members, creation time
``QuorumMember``       one replica group inside a quorum
``Timestamp``          seconds + nanoseconds
``lighthouse_main``    entry point of the stand-alone lighthouse program
=====================  ==========================================================================================
"""

from . import _ftcp as _native

__all__ = [
    "LighthouseServer",
    "LighthouseClient",
    "ManagerServer",
    "ManagerClient",
    "QuorumResult",
    "Quorum",
    "QuorumMember",
    "Timestamp",
    "lighthouse_main",
]

# re-exported under this module's name so that ``help()`` and the API reference show them here
for _name in __all__:
    globals()[_name] = getattr(_native, _name)
del _name
