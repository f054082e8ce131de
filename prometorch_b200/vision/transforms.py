"""Thirteen tensor-image transforms with the reference's names (torch/data/transforms.h): images are float tensors ``[C,H,W]``."""
import math
import random

import torch
import torch.nn.functional as F


class Compose:
    def __init__(self, ts):
        self.ts = list(ts)

    def __call__(self, x):
        for t in self.ts:
            x = t(x)
        return x


class ToTensor:
    def __call__(self, x):
        x = torch.as_tensor(x)
        if x.dtype == torch.uint8:
            x = x.float() / 255.0
        return x.permute(2, 0, 1) if x.dim() == 3 and x.shape[-1] in (1, 3, 4) and x.shape[0] not in (1, 3, 4) else x.float()


class Normalize:
    def __init__(self, mean, std):
        self.mean, self.std = torch.tensor(mean).view(-1, 1, 1), torch.tensor(std).view(-1, 1, 1)

    def __call__(self, x):
        return (x - self.mean.to(x)) / self.std.to(x)


class Resize:
    def __init__(self, size):
        self.size = (size, size) if isinstance(size, int) else tuple(size)

    def __call__(self, x):
        return F.interpolate(x[None], size=self.size, mode="bilinear", align_corners=False)[0]


class CenterCrop:
    def __init__(self, size):
        self.size = (size, size) if isinstance(size, int) else tuple(size)

    def __call__(self, x):
        h, w = x.shape[-2:]
        th, tw = self.size
        i, j = (h - th) // 2, (w - tw) // 2
        return x[..., i:i + th, j:j + tw]


class RandomCrop:
    def __init__(self, size, padding=0):
        self.size, self.padding = ((size, size) if isinstance(size, int) else tuple(size)), padding

    def __call__(self, x):
        if self.padding:
            x = F.pad(x, [self.padding] * 4)
        h, w = x.shape[-2:]
        th, tw = self.size
        i, j = random.randint(0, h - th), random.randint(0, w - tw)
        return x[..., i:i + th, j:j + tw]


class RandomHorizontalFlip:
    def __init__(self, p=0.5):
        self.p = p

    def __call__(self, x):
        return x.flip(-1) if random.random() < self.p else x


class RandomVerticalFlip(RandomHorizontalFlip):
    def __call__(self, x):
        return x.flip(-2) if random.random() < self.p else x


class Pad:
    def __init__(self, padding, fill=0.0):
        self.padding, self.fill = padding, fill

    def __call__(self, x):
        return F.pad(x, [self.padding] * 4, value=self.fill)


class RandomRotation:
    def __init__(self, degrees):
        self.degrees = degrees

    def __call__(self, x):
        a = math.radians(random.uniform(-self.degrees, self.degrees))
        theta = torch.tensor([[math.cos(a), -math.sin(a), 0.0], [math.sin(a), math.cos(a), 0.0]])[None]
        grid = F.affine_grid(theta, [1, *x.shape], align_corners=False)
        return F.grid_sample(x[None], grid, align_corners=False)[0]


class ColorJitter:
    def __init__(self, brightness=0.0, contrast=0.0):
        self.b, self.c = brightness, contrast

    def __call__(self, x):
        if self.b:
            x = x * random.uniform(1 - self.b, 1 + self.b)
        if self.c:
            m = x.mean()
            x = (x - m) * random.uniform(1 - self.c, 1 + self.c) + m
        return x.clamp(0, 1)


class Grayscale:
    def __call__(self, x):
        return (0.299 * x[0:1] + 0.587 * x[1:2] + 0.114 * x[2:3]) if x.shape[0] == 3 else x


class RandomErasing:
    def __init__(self, p=0.5, scale=(0.02, 0.2)):
        self.p, self.scale = p, scale

    def __call__(self, x):
        if random.random() >= self.p:
            return x
        h, w = x.shape[-2:]
        area = random.uniform(*self.scale) * h * w
        eh = max(1, min(h, int(math.sqrt(area))))
        ew = max(1, min(w, int(area / eh)))
        i, j = random.randint(0, h - eh), random.randint(0, w - ew)
        x = x.clone()
        x[..., i:i + eh, j:j + ew] = 0
        return x


class Lambda:
    def __init__(self, fn):
        self.fn = fn

    def __call__(self, x):
        return self.fn(x)
