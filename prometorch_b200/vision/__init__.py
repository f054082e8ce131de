"""Vision helpers: image loading (PGM / PPM natively), tensor image transforms, ``ImageFolder``, and the two
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


_PNM_EXT = (".ppm", ".pgm", ".pnm")
_PIL_EXT = (".png", ".jpg", ".jpeg", ".bmp")


def load_pnm(path: str) -> torch.Tensor:
    """A binary PGM (P5) or PPM (P6) file, or their ASCII forms (P2 / P3), as a float tensor ``[C, H, W]`` in [0, 1]."""
    with open(path, "rb") as f:
        data = f.read()
    pos, fields = 0, []
    while len(fields) < 4:                                  # magic, width, height, maximum: white space and # comments between them
        while pos < len(data) and (data[pos:pos + 1].isspace() or data[pos:pos + 1] == b"#"):
            if data[pos:pos + 1] == b"#":
                while pos < len(data) and data[pos:pos + 1] != b"\n":
                    pos += 1
            else:
                pos += 1
        start = pos
        while pos < len(data) and not data[pos:pos + 1].isspace():
            pos += 1
        if start == pos:
            raise ValueError(f"{path}: truncated PNM header")
        fields.append(data[start:pos])
    magic, w, h, maxval = fields[0], int(fields[1]), int(fields[2]), int(fields[3])
    if magic not in (b"P2", b"P3", b"P5", b"P6") or w <= 0 or h <= 0 or not 0 < maxval < 65536:
        raise ValueError(f"{path}: not a PGM / PPM file")
    c = 3 if magic in (b"P3", b"P6") else 1
    n = w * h * c
    if magic in (b"P5", b"P6"):
        pos += 1                                            # exactly one white-space byte ends the header
        width = 2 if maxval > 255 else 1
        raw = data[pos:pos + n * width]
        if len(raw) < n * width:
            raise ValueError(f"{path}: truncated pixel data")
        if width == 2:
            import numpy as np
            vals = torch.from_numpy(np.frombuffer(raw, dtype=">u2").astype("float32"))
        else:
            vals = torch.frombuffer(bytearray(raw), dtype=torch.uint8).float()
    else:
        toks = data[pos:].split()
        if len(toks) < n:
            raise ValueError(f"{path}: truncated pixel data")
        vals = torch.tensor([float(t) for t in toks[:n]])
    return (vals / maxval).view(h, w, c).permute(2, 0, 1).contiguous()


def is_supported_image(path: str) -> bool:
    return path.lower().endswith(_PNM_EXT + _PIL_EXT + (".pt", ".npy"))


def load_image(path: str) -> torch.Tensor:
    """``[C, H, W]`` float in [0, 1]: PGM / PPM natively, PNG / JPEG / BMP through Pillow when it is installed, tensors saved
    as ``.pt`` / ``.npy`` as they are (torch/vision/vision.h:85-160)."""
    low = path.lower()
    if low.endswith(_PNM_EXT):
        return load_pnm(path)
    if low.endswith(".npy"):
        import numpy as np
        return torch.from_numpy(np.load(path)).float()
    if low.endswith(".pt"):
        return torch.load(path, weights_only=True).float()
    if low.endswith(_PIL_EXT):
        try:
            from PIL import Image
        except ImportError as e:
            raise RuntimeError(f"{path}: reading this format needs Pillow; PGM / PPM files are read natively") from e
        import numpy as np
        img = np.asarray(Image.open(path).convert("RGB"), dtype="float32") / 255.0
        return torch.from_numpy(img).permute(2, 0, 1).contiguous()
    raise ValueError(f"{path}: unsupported image format")


def save_pnm(path: str, x: torch.Tensor):
    """``[C, H, W]`` (C = 1 or 3) in [0, 1] as a binary PGM / PPM file."""
    c, h, w = x.shape
    assert c in (1, 3), "PGM holds one channel, PPM three"
    raw = (x.clamp(0, 1) * 255 + 0.5).to(torch.uint8).permute(1, 2, 0).contiguous().numpy().tobytes()
    with open(path, "wb") as f:
        f.write(b"P6\n" if c == 3 else b"P5\n")
        f.write(f"{w} {h}\n255\n".encode())
        f.write(raw)


class ImageFolder(torch.utils.data.Dataset):
    """``root/<class>/<file>``: image files (PGM / PPM, PNG / JPEG with Pillow) or tensors ``[C, H, W]`` saved as ``.pt`` / ``.npy``."""

    def __init__(self, root: str, transform: Optional[Callable] = None):
        self.classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        self.class_to_idx = {c: i for i, c in enumerate(self.classes)}
        self.samples = [(os.path.join(root, c, f), i) for i, c in enumerate(self.classes) for f in sorted(os.listdir(os.path.join(root, c)))
                        if is_supported_image(f)]
        self.transform = transform

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        p, y = self.samples[i]
        x = load_image(p)
        return (self.transform(x) if self.transform else x), y


class ConvBNReLU(nn.Sequential):
    """Convolution + batch norm + ReLU6, the building block of MobileNetV2 (torch/vision/models.h:51)."""

    def __init__(self, i: int, o: int, kernel: int = 3, stride: int = 1, groups: int = 1):
        super().__init__(nn.Conv2d(i, o, kernel, stride, (kernel - 1) // 2, groups=groups, bias=False), nn.BatchNorm2d(o), nn.ReLU6(inplace=True))


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
