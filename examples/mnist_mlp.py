#!/usr/bin/env python
"""MNIST-style MLP classifier with the promethorch API (the counterpart of examples/mnist/train_mnist_mlp.cpp).

    python examples/mnist_mlp.py [--data DIR] [--epochs 2] [--device cpu|cuda]

``--data DIR`` reads the four IDX files of MNIST (train-images-idx3-ubyte ...); without it the script trains on a
synthetic set of the same shape (ten noisy class prototypes), since no dataset ships with the package.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import promethorch as pt  # noqa: E402


def load(data_dir, n_train, n_test):
    if data_dir:                        # the four IDX files of MNIST / Fashion-MNIST (optionally .gz)
        from prometorch_b200.data import MNIST
        tr, te = MNIST(data_dir, train=True, flatten=True), MNIST(data_dir, train=False, flatten=True)
        return tr.images.reshape(-1, 784), tr.labels, te.images.reshape(-1, 784), te.labels
    pt.manual_seed(1234)
    protos = pt.rand(10, 784)

    def make(n):
        y = pt.randint(0, 10, (n,))
        return (protos[y] + 0.8 * pt.randn(n, 784)).clamp(0, 1), y
    return (*make(n_train), *make(n_test))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default=None)
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--samples", type=int, default=20000)
    ap.add_argument("--save", default=None, help="write the trained weights to this file (PTOR container)")
    a = ap.parse_args()
    xtr, ytr, xte, yte = load(a.data, a.samples, 2000)
    model = pt.nn.Sequential(pt.nn.Linear(784, 512), pt.nn.ReLU(), pt.nn.Linear(512, 256), pt.nn.ReLU(), pt.nn.Linear(256, 10)).to(a.device)
    opt = pt.optim.Adam(model.parameters(), lr=1e-3)
    sched = pt.optim.StepLR(opt, step_size=1, gamma=0.7)
    loader = pt.data.DataLoader(pt.data.TensorDataset(xtr, ytr), batch_size=a.batch, shuffle=True)
    loss_fn = pt.nn.CrossEntropyLoss()
    for epoch in range(a.epochs):
        model.train()
        for x, y in loader:
            opt.zero_grad()
            loss = loss_fn(model(x.to(a.device)), y.to(a.device))
            loss.backward()
            opt.step()
        sched.step()
        model.eval()
        with pt.no_grad():
            acc = float((model(xte.to(a.device)).argmax(-1).cpu() == yte).float().mean())
        print(f"epoch {epoch + 1}: loss {float(loss):.4f}  test accuracy {100 * acc:.2f} %  lr {sched.get_last_lr():.2e}")
    if a.save:
        pt.save(model.state_dict(), a.save)
        print("saved", a.save)


if __name__ == "__main__":
    main()
