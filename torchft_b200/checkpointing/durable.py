"""Durable (on-disk) checkpoints next to live recovery.

Live recovery (the checkpoint transports) repairs a job that lost some replica groups; a durable
checkpoint is what brings a job back after *all* of them are gone.  The reference leaves it to the
user ("periodically checkpoint model, optim, manager and dataloader", train_ddp.py:201-208) and only
provides ``Manager.state_dict()/load_state_dict()`` (torchft/manager.py:880-912); this module is
that piece, written once.

Layout: ``<dir>/step_<NNNNNNNN>/rank_<R>.pt`` holds, for one rank of one replica group, the same
nesting that healing transfers, ``{"user": {key: state}, "torchft": {"step", "batches_committed"}}``,
plus whatever ``extra`` the caller passes (data-loader position, RNG state).  A file is written to a
temporary name and renamed, so a crash never leaves a half-written checkpoint under its final name;
a step counts as complete when every rank's file exists.  Only one replica group needs to write
(they hold identical state after every committed step).
"""

from __future__ import annotations

import os
import re
import shutil
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ..manager import Manager

_STEP_RE = re.compile(r"^step_(\d{8})$")


class DurableCheckpointer:
    """Writes and restores on-disk checkpoints of everything registered with a :class:`Manager` (user state, step and
    batch counters, caller-supplied extras); see the module docstring for the layout."""

    def __init__(self, manager: Manager, directory: str, rank: int, world_size: int, every: int = 0, keep: int = 2) -> None:
        """``rank`` / ``world_size``: this rank's position inside its replica group.  ``every``:
        :meth:`maybe_save` writes when the committed step is a multiple of it (0 = never).
        ``keep``: complete checkpoints retained (older ones are removed by group rank 0)."""
        self.manager, self.dir = manager, Path(directory)
        self.rank, self.world_size, self.every, self.keep = rank, world_size, every, max(1, keep)
        self._last_saved = -1

    # ------------------------------------------------------------------ writing
    def save(self, extra: Optional[Dict[str, object]] = None) -> Path:
        """Write this rank's state for the manager's current step; returns the file."""
        manager = self.manager
        step = manager.current_step()
        payload = {
            "user": {key: fn() for key, fn in manager._user_state_dicts.items()},
            "torchft": manager.state_dict(),
            "extra": extra or {},
        }
        d = self.dir / f"step_{step:08d}"
        d.mkdir(parents=True, exist_ok=True)
        final = d / f"rank_{self.rank}.pt"
        tmp = d / f".rank_{self.rank}.pt.tmp{os.getpid()}"
        torch.save(payload, tmp)
        os.replace(tmp, final)
        self._last_saved = step
        if self.rank == 0:
            self._prune()
        return final

    def maybe_save(self, extra: Optional[Dict[str, object]] = None) -> Optional[Path]:
        """Call after every step: saves once per committed step that is a multiple of ``every``."""
        step = self.manager.current_step()
        if self.every > 0 and step > 0 and step % self.every == 0 and step != self._last_saved:
            return self.save(extra)
        return None

    def _prune(self) -> None:
        done = self.complete_steps()
        for step in done[: -self.keep]:
            shutil.rmtree(self.dir / f"step_{step:08d}", ignore_errors=True)

    # ------------------------------------------------------------------ reading
    def complete_steps(self) -> List[int]:
        """Steps for which every rank of the group has written its file, ascending."""
        if not self.dir.is_dir():
            return []
        steps = []
        for child in self.dir.iterdir():
            m = _STEP_RE.match(child.name)
            if m and all((child / f"rank_{r}.pt").is_file() for r in range(self.world_size)):
                steps.append(int(m.group(1)))
        return sorted(steps)

    def load_latest(self) -> Optional[Dict[str, object]]:
        """Restore the newest complete checkpoint into the registered state and the manager
        (step, batches_committed).  Returns the ``extra`` dict that was saved with it, or None
        when there is no complete checkpoint.  Call before the first step."""
        steps = self.complete_steps()
        if not steps:
            return None
        payload = torch.load(self.dir / f"step_{steps[-1]:08d}" / f"rank_{self.rank}.pt", weights_only=False)
        user = payload["user"]
        for key, load in self.manager._load_state_dict_fns.items():
            load(user[key])
        self.manager.load_state_dict(payload["torchft"])
        self._last_saved = int(payload["torchft"]["step"])
        return payload.get("extra", {})
