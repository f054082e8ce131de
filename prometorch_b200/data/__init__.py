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
