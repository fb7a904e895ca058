"""Guard zones around kernel outputs: a tensor is carved out of a larger byte buffer whose
margins hold a fixed pattern, and the margins are compared after the kernels ran.  Catches
out-of-bounds writes of the production build without any tool."""
from typing import List, Tuple

import torch

GUARD = 4096  # bytes on each side; a multiple of every alignment the kernels ask for
PATTERN = 0xA5


class Canaries:
    def __init__(self, device) -> None:
        self.device = device
        self._bufs: List[Tuple[str, torch.Tensor, int]] = []

    def empty(self, shape, dtype, name: str = "") -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        pad = (-nbytes) % 256
        raw = torch.full((GUARD + nbytes + pad + GUARD,), PATTERN, dtype=torch.uint8, device=self.device)
        self._bufs.append((name or f"buf{len(self._bufs)}", raw, nbytes))
        return raw[GUARD : GUARD + nbytes].view(dtype).view(*shape)

    def like(self, t: torch.Tensor, name: str = "") -> torch.Tensor:
        out = self.empty(tuple(t.shape), t.dtype, name)
        out.copy_(t)
        return out

    def check(self) -> None:
        torch.cuda.synchronize()
        for name, raw, nbytes in self._bufs:
            head = raw[:GUARD]
            tail = raw[GUARD + nbytes :]
            assert bool((head == PATTERN).all()), f"{name}: bytes before the tensor were overwritten"
            assert bool((tail == PATTERN).all()), f"{name}: bytes after the tensor were overwritten"
