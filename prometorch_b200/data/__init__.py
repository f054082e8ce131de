"""Datasets, samplers, ``DataLoader`` and the distributed sampler (torch/data/*.h in the reference).

``torch.utils.data`` supplies the loader machinery (worker processes, prefetching, pinned memory);
``DistributedSampler`` has the reference's semantics, which are PyTorch's: seed+epoch shuffle, pad or
drop to a multiple of the world size, then ``indices[rank::world]`` (torch/data/distributed_sampler.h:1-80)."""
from torch.utils.data import (BatchSampler, ConcatDataset, DataLoader, Dataset, IterableDataset, RandomSampler, Sampler,
                              SequentialSampler, Subset, SubsetRandomSampler, TensorDataset, WeightedRandomSampler, random_split)
from torch.utils.data.distributed import DistributedSampler

import torch


class MapDataset(Dataset):
    """Applies ``fn`` to every sample of ``dataset`` (the reference's ``MapDataset``)."""

    def __init__(self, dataset, fn):
        self.dataset, self.fn = dataset, fn

    def __len__(self):
        return len(self.dataset)

    def __getitem__(self, i):
        return self.fn(self.dataset[i])


class SyntheticTokens(Dataset):
    """Uniform-random token sequences of a fixed shape — the data of the benchmark configs."""

    def __init__(self, n: int, seq_len: int, vocab: int, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.x = torch.randint(0, vocab, (n, seq_len + 1), generator=g)

    def __len__(self):
        return self.x.shape[0]

    def __getitem__(self, i):
        return self.x[i, :-1], self.x[i, 1:]


class SyntheticImages(Dataset):
    """28x28 "images" with pixels uniform in [0,1], flattened to 784, labels uniform in 0..9."""

    def __init__(self, n: int = 60000, seed: int = 0, dim: int = 784, classes: int = 10):
        g = torch.Generator().manual_seed(seed)
        self.x = torch.rand(n, dim, generator=g)
        self.y = torch.randint(0, classes, (n,), generator=g)

    def __len__(self):
        return self.x.shape[0]

    def __getitem__(self, i):
        return self.x[i], self.y[i]


def read_idx(path: str) -> torch.Tensor:
    """An IDX file (the MNIST container: magic ``00 00 <dtype> <ndim>``, big-endian dims, raw data; ``.gz`` accepted)
    as a tensor.  The reference's MNIST programs parse the same files by hand (examples/mnist/train_mnist_mlp.cpp)."""
    import gzip
    import struct
    import numpy as np
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rb") as f:
        raw = f.read()
    zero, dtype_code, ndim = struct.unpack(">HBB", raw[:4])
    if zero != 0:
        raise ValueError(f"{path}: not an IDX file")
    dtypes = {0x08: np.uint8, 0x09: np.int8, 0x0B: np.dtype(">i2"), 0x0C: np.dtype(">i4"), 0x0D: np.dtype(">f4"), 0x0E: np.dtype(">f8")}
    if dtype_code not in dtypes:
        raise ValueError(f"{path}: unknown IDX element type {dtype_code:#x}")
    dims = struct.unpack(">" + "I" * ndim, raw[4:4 + 4 * ndim])
    arr = np.frombuffer(raw, dtype=dtypes[dtype_code], offset=4 + 4 * ndim)
    n = 1
    for d in dims:
        n *= d
    if arr.size != n:
        raise ValueError(f"{path}: {arr.size} elements, header says {dims}")
    return torch.from_numpy(arr.astype(arr.dtype.newbyteorder("=")).reshape(dims).copy())


class MNIST(Dataset):
    """MNIST / Fashion-MNIST from the four IDX files in ``root`` (``train-images-idx3-ubyte`` ..., optionally ``.gz``):
    images as float ``[1, 28, 28]`` in [0, 1] (or flattened), labels as int64."""

    def __init__(self, root: str, train: bool = True, flatten: bool = False, transform=None):
        import os
        stem = "train" if train else "t10k"

        def find(name):
            for cand in (name, name + ".gz", name.replace("-idx", ".idx"), name.replace("-idx", ".idx") + ".gz"):
                p = os.path.join(root, cand)
                if os.path.exists(p):
                    return p
            raise FileNotFoundError(f"{name}[.gz] not found under {root}")
        self.images = read_idx(find(f"{stem}-images-idx3-ubyte")).float().div_(255.0)
        self.labels = read_idx(find(f"{stem}-labels-idx1-ubyte")).long()
        if self.images.shape[0] != self.labels.shape[0]:
            raise ValueError("MNIST: image and label counts differ")
        self.flatten, self.transform = flatten, transform

    def __len__(self):
        return self.images.shape[0]

    def __getitem__(self, i):
        x = self.images[i]
        x = x.reshape(-1) if self.flatten else x.unsqueeze(0)
        if self.transform is not None:
            x = self.transform(x)
        return x, self.labels[i]


class CharTextDataset(Dataset):
    """Character-level language-model samples from a text file: windows of ``block_size + 1`` characters, split into
    input and next-character target (the data of the reference's shakespeare example)."""

    def __init__(self, path_or_text: str, block_size: int = 128, stride: int = 1, is_text: bool = False):
        text = path_or_text if is_text else open(path_or_text, encoding="utf-8").read()
        self.chars = sorted(set(text))
        self.stoi = {c: i for i, c in enumerate(self.chars)}
        self.data = torch.tensor([self.stoi[c] for c in text], dtype=torch.long)
        self.block_size, self.stride = block_size, stride
        if self.data.numel() <= block_size:
            raise ValueError("CharTextDataset: the text is shorter than one block")

    @property
    def vocab_size(self) -> int:
        return len(self.chars)

    def decode(self, ids) -> str:
        return "".join(self.chars[int(i)] for i in ids)

    def __len__(self):
        return (self.data.numel() - self.block_size - 1) // self.stride + 1

    def __getitem__(self, i):
        s = i * self.stride
        w = self.data[s:s + self.block_size + 1]
        return w[:-1], w[1:]


# ---------------------------------------------------------------------------------------------- the reference's helper names (torch/data/*.h)
from dataclasses import dataclass as _dataclass  # noqa: E402
from typing import Any as _Any, Callable as _Callable, Optional as _Optional, Sequence as _Sequence  # noqa: E402


@_dataclass
class DataLoaderOptions:
    """The fields of the reference's options struct; ``make_loader(dataset, options)`` builds a loader from them."""
    batch_size: int = 1
    shuffle: bool = False
    num_workers: int = 0
    prefetch_factor: int = 2
    drop_last: bool = False
    pin_memory: bool = False
    seed: _Optional[int] = None


def make_loader(dataset, options: DataLoaderOptions = None, sampler=None, collate_fn=None) -> DataLoader:
    o = options or DataLoaderOptions()
    gen = torch.Generator().manual_seed(o.seed) if o.seed is not None else None
    return DataLoader(dataset, batch_size=o.batch_size, shuffle=o.shuffle and sampler is None, sampler=sampler, num_workers=o.num_workers,
                      prefetch_factor=o.prefetch_factor if o.num_workers > 0 else None, drop_last=o.drop_last, pin_memory=o.pin_memory,
                      generator=gen, collate_fn=collate_fn)


@_dataclass
class Example:
    """One sample: data and target."""
    data: _Any
    target: _Any = None


@_dataclass
class Batch:
    """A collated batch: ``data [B, ...]`` and ``target [B, ...]``."""
    data: torch.Tensor
    target: _Optional[torch.Tensor] = None

    def to(self, device, non_blocking: bool = False) -> "Batch":
        return Batch(self.data.to(device, non_blocking=non_blocking), None if self.target is None else self.target.to(device, non_blocking=non_blocking))

    def __iter__(self):
        return iter((self.data, self.target))


class DefaultCollate:
    """Stack ``Example``s or ``(data, target)`` pairs into a :class:`Batch`."""

    def __call__(self, samples) -> Batch:
        pairs = [(s.data, s.target) if isinstance(s, Example) else (s if isinstance(s, (tuple, list)) else (s, None)) for s in samples]
        data = torch.stack([torch.as_tensor(d) for d, _ in pairs])
        target = None if pairs[0][1] is None else torch.stack([torch.as_tensor(t) for _, t in pairs])
        return Batch(data, target)


class Transform:
    def __call__(self, x):
        raise NotImplementedError


class Compose(Transform):
    def __init__(self, transforms: _Sequence[_Callable]):
        self.transforms = list(transforms)

    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class Lambda(Transform):
    def __init__(self, fn: _Callable):
        self.fn = fn

    def __call__(self, x):
        return self.fn(x)


class Normalize(Transform):
    """``(x - mean) / std`` with scalars or per-channel values (broadcast over the trailing dimensions)."""

    def __init__(self, mean, std):
        self.mean, self.std = torch.as_tensor(mean, dtype=torch.float32), torch.as_tensor(std, dtype=torch.float32)

    def __call__(self, x):
        m, s = self.mean, self.std
        if m.dim() == 1 and x.dim() > 1:
            shape = [-1] + [1] * (x.dim() - 1)
            m, s = m.view(shape), s.view(shape)
        return (x - m) / s


class Flatten(Transform):
    def __call__(self, x):
        return x.reshape(-1)


def make_sequential_sampler(dataset) -> Sampler:
    return SequentialSampler(dataset)


def make_random_sampler(dataset, seed: _Optional[int] = None) -> Sampler:
    return RandomSampler(dataset, generator=torch.Generator().manual_seed(seed) if seed is not None else None)


def make_batch_sampler(sampler, batch_size: int, drop_last: bool = False) -> BatchSampler:
    return BatchSampler(sampler, batch_size, drop_last)
