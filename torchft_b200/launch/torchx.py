"""torchx component: one ``torchrun`` role per replica group.

    torchx run -- torchft_b200/launch/torchx.py:hsdp --replicas 2 --workers_per_replica 4 train_hsdp.py

Each role gets ``REPLICA_GROUP_ID``, ``NUM_REPLICA_GROUPS``, ``TORCHFT_LIGHTHOUSE`` and its
own ``--master_port`` (29600 + group id) and restarts up to ``max_restarts`` times
(shape of torchft/torchx.py:11-83).  torchx is optional: importing this module without it
raises only when the component is actually called.
"""

from __future__ import annotations

import os
from typing import Dict, Optional


def hsdp(*script_args: str, replicas: int = 2, workers_per_replica: int = 1, max_restarts: int = 10,
         script: str = "train_ddp.py", env: Optional[Dict[str, str]] = None, image: str = "", h: Optional[str] = None,
         cpu: int = 2, gpu: int = 0, memMB: int = 1024):
    """torchx component: an ``AppDef`` with one ``torchrun`` role per replica group (``replicas`` groups of
    ``workers_per_replica`` workers), each with ``REPLICA_GROUP_ID``, ``NUM_REPLICA_GROUPS`` and ``TORCHFT_LIGHTHOUSE`` in
    its environment, its own ``--master_port`` (29600 + group) and ``--max_restarts`` (torchft/torchx.py:11-83)."""
    try:
        import torchx.specs as specs
    except ImportError as e:  # pragma: no cover - torchx is not a dependency
        raise RuntimeError("the torchx launcher needs the `torchx` package") from e
    env = dict(env or {})
    env.setdefault("TORCHFT_LIGHTHOUSE", os.environ.get("TORCHFT_LIGHTHOUSE", "http://localhost:29510"))
    env["TORCHX_TRACKING_EXPERIMENT_NAME"] = "torchft_b200"
    roles = []
    for g in range(replicas):
        roles.append(
            specs.Role(
                name=f"replica_{g}", image=image, min_replicas=workers_per_replica, num_replicas=workers_per_replica,
                resource=specs.resource(cpu=cpu, gpu=gpu, memMB=memMB, h=h), max_retries=max_restarts,
                env={**env, "REPLICA_GROUP_ID": str(g), "NUM_REPLICA_GROUPS": str(replicas)},
                entrypoint="torchrun",
                args=["--rdzv_backend=c10d", "--rdzv_endpoint=localhost:0", f"--max_restarts={max_restarts}",
                      "--nnodes=1", f"--nproc_per_node={workers_per_replica}", f"--master_port={29600 + g}", script,
                      *script_args],
            )
        )
    return specs.AppDef(name="torchft_b200", roles=roles)
