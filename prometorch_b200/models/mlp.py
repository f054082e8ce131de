"""The MLP classifier of the CPU benchmark config: 784 -> 512 -> 256 -> 10 with ReLU."""
import torch.nn as nn


class MLPClassifier(nn.Sequential):
    def __init__(self, sizes=(784, 512, 256, 10)):
        layers = []
        for i, (a, b) in enumerate(zip(sizes[:-1], sizes[1:])):
            layers.append(nn.Linear(a, b))
            if i < len(sizes) - 2:
                layers.append(nn.ReLU())
        super().__init__(*layers)
