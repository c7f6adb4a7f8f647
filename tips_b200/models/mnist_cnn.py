"""The MNIST-shaped CNN of the reference's Keras example
(examples/tensorflow2_keras_mnist.py:45-60): conv3x3x32-relu, conv3x3x64-relu,
maxpool2, dropout, dense128-relu, dropout, dense10.  Used on CPU ranks to
exercise DistributedOptimizer end to end."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class MnistCNN(nn.Module):
    def __init__(self, dropout: bool = False):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 32, 3)
        self.conv2 = nn.Conv2d(32, 64, 3)
        self.drop1 = nn.Dropout(0.25) if dropout else nn.Identity()
        self.fc1 = nn.Linear(64 * 12 * 12, 128)
        self.drop2 = nn.Dropout(0.5) if dropout else nn.Identity()
        self.fc2 = nn.Linear(128, 10)

    def forward(self, x):
        x = F.relu(self.conv1(x))
        x = F.relu(self.conv2(x))
        x = self.drop1(F.max_pool2d(x, 2))
        x = torch.flatten(x, 1)
        x = self.drop2(F.relu(self.fc1(x)))
        return self.fc2(x)


def synthetic_batch(batch: int, seed: int, device="cpu"):
    """28x28x1 inputs uniform in [0,1], labels uniform in 0..9."""
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(batch, 1, 28, 28, generator=g)
    y = torch.randint(0, 10, (batch,), generator=g)
    return x.to(device), y.to(device)
