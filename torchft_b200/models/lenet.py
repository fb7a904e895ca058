"""LeNet-style CNN used by the DDP example and the CPU integration tests: conv 3->6 k5,
maxpool 2, conv 6->16 k5, maxpool 2, fc 400->120->84->10, ReLU, for 3x32x32 inputs."""

import torch
from torch import nn


class LeNet(nn.Module):
    def __init__(self, num_classes: int = 10) -> None:
        super().__init__()
        self.cnn = nn.Sequential(
            nn.Conv2d(3, 6, 5), nn.ReLU(), nn.MaxPool2d(2, 2), nn.Conv2d(6, 16, 5), nn.ReLU(), nn.MaxPool2d(2, 2)
        )
        self.classifier = nn.Sequential(
            nn.Linear(16 * 5 * 5, 120), nn.ReLU(), nn.Linear(120, 84), nn.ReLU(), nn.Linear(84, num_classes)
        )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.classifier(torch.flatten(self.cnn(x), 1))


def synthetic_batch(batch: int, seed: int, device="cpu"):
    """Seeded N(0,1) images and uniform labels."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(batch, 3, 32, 32, generator=g).to(device), torch.randint(0, 10, (batch,), generator=g).to(device)
