"""Vision helpers: tensor image transforms, ``ImageFolder``-style dataset over ``.pt``/``.npy`` trees, and the two
reference CNNs (MobileNetV2, CIFAR ResNet-20; torch/vision/*.h)."""
from __future__ import annotations

import math
import os
import random
from typing import Callable, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import transforms  # noqa: F401


class ImageFolder(torch.utils.data.Dataset):
    """``root/<class>/<file>`` where files are tensors saved with ``torch.save`` or ``.npy`` arrays ``[C,H,W]``."""

    def __init__(self, root: str, transform: Optional[Callable] = None):
        self.classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        self.samples = [(os.path.join(root, c, f), i) for i, c in enumerate(self.classes) for f in sorted(os.listdir(os.path.join(root, c)))
                        if f.endswith((".pt", ".npy"))]
        self.transform = transform

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        p, y = self.samples[i]
        if p.endswith(".npy"):
            import numpy as np
            x = torch.from_numpy(np.load(p)).float()
        else:
            x = torch.load(p, weights_only=True).float()
        return (self.transform(x) if self.transform else x), y


class _InvertedResidual(nn.Module):
    def __init__(self, i, o, stride, expand):
        super().__init__()
        h = i * expand
        self.use_res = stride == 1 and i == o
        layers = []
        if expand != 1:
            layers += [nn.Conv2d(i, h, 1, bias=False), nn.BatchNorm2d(h), nn.ReLU6(inplace=True)]
        layers += [nn.Conv2d(h, h, 3, stride, 1, groups=h, bias=False), nn.BatchNorm2d(h), nn.ReLU6(inplace=True),
                   nn.Conv2d(h, o, 1, bias=False), nn.BatchNorm2d(o)]
        self.conv = nn.Sequential(*layers)

    def forward(self, x):
        return x + self.conv(x) if self.use_res else self.conv(x)


class MobileNetV2(nn.Module):
    def __init__(self, num_classes: int = 1000, width: float = 1.0):
        super().__init__()
        cfg = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
        c = int(32 * width)
        feats = [nn.Conv2d(3, c, 3, 2, 1, bias=False), nn.BatchNorm2d(c), nn.ReLU6(inplace=True)]
        for t, o, n, s in cfg:
            o = int(o * width)
            for k in range(n):
                feats.append(_InvertedResidual(c, o, s if k == 0 else 1, t))
                c = o
        last = int(1280 * max(1.0, width))
        feats += [nn.Conv2d(c, last, 1, bias=False), nn.BatchNorm2d(last), nn.ReLU6(inplace=True)]
        self.features = nn.Sequential(*feats)
        self.classifier = nn.Linear(last, num_classes)

    def forward(self, x):
        return self.classifier(self.features(x).mean((2, 3)))


class _BasicBlock(nn.Module):
    def __init__(self, i, o, stride):
        super().__init__()
        self.c1, self.b1 = nn.Conv2d(i, o, 3, stride, 1, bias=False), nn.BatchNorm2d(o)
        self.c2, self.b2 = nn.Conv2d(o, o, 3, 1, 1, bias=False), nn.BatchNorm2d(o)
        self.short = None if stride == 1 and i == o else nn.Sequential(nn.Conv2d(i, o, 1, stride, bias=False), nn.BatchNorm2d(o))

    def forward(self, x):
        y = self.b2(self.c2(F.relu(self.b1(self.c1(x)))))
        return F.relu(y + (x if self.short is None else self.short(x)))


class ResNet20(nn.Module):
    """CIFAR ResNet-20: 3 stages x 3 basic blocks, 16/32/64 channels."""

    def __init__(self, num_classes: int = 10):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, 16, 3, 1, 1, bias=False), nn.BatchNorm2d(16), nn.ReLU(inplace=True))
        blocks, c = [], 16
        for o, s in ((16, 1), (32, 2), (64, 2)):
            for k in range(3):
                blocks.append(_BasicBlock(c, o, s if k == 0 else 1))
                c = o
        self.layers = nn.Sequential(*blocks)
        self.fc = nn.Linear(64, num_classes)

    def forward(self, x):
        return self.fc(self.layers(self.stem(x)).mean((2, 3)))
