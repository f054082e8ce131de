#!/usr/bin/env python
"""Ten small models trained end to end with the promethorch API: the model zoo of the reference's
examples/train_10_models.cpp (linear and logistic regression, XOR, three MNIST-shaped MLPs, RNN / LSTM / GRU cells on
sequence tasks, and a save / load round trip), each with the optimizer the reference uses for it.

    python examples/train_10_models.py [--quick] [--device cpu|cuda] [--only N]

No dataset ships with the package: the MNIST-shaped tasks use ten noisy class prototypes (pass real MNIST through
examples/mnist_mlp.py --data).  Every task prints its final metric and PASS / FAIL against a threshold; the exit code is
the number of failures.
"""
import argparse
import math
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import promethorch as pt  # noqa: E402

nn = pt.nn


def mnist_like(n, seed, noise=0.8):
    g = pt.Generator().manual_seed(1234)
    protos = pt.rand(10, 784, generator=g)
    g2 = pt.Generator().manual_seed(seed)
    y = pt.randint(0, 10, (n,), generator=g2)
    return (protos[y] + noise * pt.randn(n, 784, generator=g2)).clamp(0, 1), y


def fit_classifier(model, opt, x, y, epochs, batch, dev):
    loss_fn = nn.CrossEntropyLoss()
    loader = pt.data.DataLoader(pt.data.TensorDataset(x, y), batch_size=batch, shuffle=True)
    model.train()
    for _ in range(epochs):
        for xb, yb in loader:
            opt.zero_grad()
            loss_fn(model(xb.to(dev)), yb.to(dev)).backward()
            opt.step()
    model.eval()


def accuracy(model, x, y, dev):
    with pt.no_grad():
        return float((model(x.to(dev)).argmax(-1).cpu() == y).float().mean())


# ----------------------------------------------------------------------------------------------------------- the ten
def linear_regression(a):
    """y = 3 x1 + 2 x2 - 1 + noise, MSE, SGD."""
    x = pt.randn(512, 2)
    y = 3 * x[:, :1] + 2 * x[:, 1:] - 1 + 0.05 * pt.randn(512, 1)
    m = nn.Linear(2, 1).to(a.device)
    opt = pt.optim.SGD(m.parameters(), lr=0.1)
    for _ in range(a.steps(200)):
        opt.zero_grad()
        loss = nn.functional.mse_loss(m(x.to(a.device)), y.to(a.device))
        loss.backward()
        opt.step()
    w, b = m.weight.detach().cpu().flatten().tolist(), float(m.bias.detach())
    return "final MSE", loss.item(), loss.item() < 0.02 and abs(w[0] - 3) < 0.1 and abs(w[1] - 2) < 0.1 and abs(b + 1) < 0.1


def logistic_regression(a):
    """Inside / outside the unit circle from (x1^2, x2^2), BCE, SGD."""
    x = pt.rand(1024, 2) * 3 - 1.5
    y = ((x ** 2).sum(1, keepdim=True) < 1).float()
    m = nn.Sequential(nn.Linear(2, 1), nn.Sigmoid()).to(a.device)
    opt = pt.optim.SGD(m.parameters(), lr=1.0)
    f = (x ** 2).to(a.device)
    for _ in range(a.steps(400)):
        opt.zero_grad()
        loss = nn.functional.binary_cross_entropy(m(f), y.to(a.device))
        loss.backward()
        opt.step()
    acc = float(((m(f) > 0.5).float().cpu() == y).float().mean())
    return "accuracy", acc, acc > 0.93


def xor_mlp(a):
    """Two-layer MLP on the four XOR points, MSE, Adam."""
    x = pt.tensor([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]])
    y = pt.tensor([[0.0], [1.0], [1.0], [0.0]])
    m = nn.Sequential(nn.Linear(2, 8), nn.Tanh(), nn.Linear(8, 1), nn.Sigmoid()).to(a.device)
    opt = pt.optim.Adam(m.parameters(), lr=0.05)
    for _ in range(a.steps(600)):
        opt.zero_grad()
        loss = nn.functional.mse_loss(m(x.to(a.device)), y.to(a.device))
        loss.backward()
        opt.step()
    return "final MSE", loss.item(), loss.item() < 0.02


def simple_mnist(a):
    """784 -> 128 -> 10, SGD lr 0.01 with momentum."""
    x, y = mnist_like(a.samples, 1)
    xt, yt = mnist_like(2000, 2)
    m = nn.Sequential(nn.Linear(784, 128), nn.ReLU(), nn.Linear(128, 10)).to(a.device)
    fit_classifier(m, pt.optim.SGD(m.parameters(), lr=0.01, momentum=0.9), x, y, a.epochs, 64, a.device)
    acc = accuracy(m, xt, yt, a.device)
    return "test accuracy", acc, acc > 0.9


def deep_mnist(a):
    """784 -> 512 -> 256 -> 128 -> 10, Adam lr 0.001."""
    x, y = mnist_like(a.samples, 3)
    xt, yt = mnist_like(2000, 4)
    m = nn.Sequential(nn.Linear(784, 512), nn.ReLU(), nn.Linear(512, 256), nn.ReLU(), nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 10)).to(a.device)
    fit_classifier(m, pt.optim.Adam(m.parameters(), lr=1e-3), x, y, a.epochs, 64, a.device)
    acc = accuracy(m, xt, yt, a.device)
    return "test accuracy", acc, acc > 0.9


def dropout_mnist(a):
    """784 -> 256 -> 128 -> 10 with dropout 0.2, AdamW + cosine schedule."""
    x, y = mnist_like(a.samples, 5)
    xt, yt = mnist_like(2000, 6)
    m = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Dropout(0.2), nn.Linear(256, 128), nn.ReLU(), nn.Dropout(0.2), nn.Linear(128, 10)).to(a.device)
    opt = pt.optim.AdamW(m.parameters(), lr=2e-3, weight_decay=0.01)
    sched = pt.optim.CosineAnnealingLR(opt, T_max=a.epochs)
    for _ in range(a.epochs):
        fit_classifier(m, opt, x, y, 1, 64, a.device)
        sched.step()
    acc = accuracy(m, xt, yt, a.device)
    return "test accuracy", acc, acc > 0.9


class CellNet(nn.Module):
    """A recurrent cell unrolled over the sequence, then a linear read-out of the last hidden state."""

    def __init__(self, kind, inp, hidden, out):
        super().__init__()
        self.kind, self.hidden = kind, hidden
        self.cell = {"rnn": nn.RNNCell, "lstm": nn.LSTMCell, "gru": nn.GRUCell}[kind](inp, hidden)
        self.fc = nn.Linear(hidden, out)

    def forward(self, x):                                   # [B, T, inp]
        h = x.new_zeros(x.shape[0], self.hidden)
        c = x.new_zeros(x.shape[0], self.hidden)
        for t in range(x.shape[1]):
            if self.kind == "lstm":
                h, c = self.cell(x[:, t], (h, c))
            else:
                h = self.cell(x[:, t], h)
        return self.fc(h)


def rnn_sine(a):
    """Next value of a sine wave from the previous 20, RNNCell + Linear, Adam."""
    t0 = pt.rand(256, 1) * 2 * math.pi
    steps = pt.arange(21).float() * 0.3
    wave = pt.sin(t0 + steps)
    x, y = wave[:, :20].unsqueeze(-1), wave[:, 20:]
    m = CellNet("rnn", 1, 32, 1).to(a.device)
    opt = pt.optim.Adam(m.parameters(), lr=0.01)
    for _ in range(a.steps(300)):
        opt.zero_grad()
        loss = nn.functional.mse_loss(m(x.to(a.device)), y.to(a.device))
        loss.backward()
        pt.nn.utils.clip_grad_norm_(m.parameters(), 1.0)
        opt.step()
    return "final MSE", loss.item(), loss.item() < 0.02


def lstm_sequence(a):
    """Is the sum of a 12-step sequence positive?  LSTMCell + Linear, Adam."""
    x = pt.randn(1024, 12, 1)
    y = (x.sum((1, 2)) > 0).long()
    m = CellNet("lstm", 1, 32, 2).to(a.device)
    opt = pt.optim.Adam(m.parameters(), lr=0.01)
    for _ in range(a.steps(150)):
        opt.zero_grad()
        nn.functional.cross_entropy(m(x.to(a.device)), y.to(a.device)).backward()
        opt.step()
    acc = accuracy(m, x, y, a.device)
    return "accuracy", acc, acc > 0.9


def gru_trend(a):
    """Rising or falling noisy ramp, GRUCell + Linear, RMSprop."""
    slope = pt.randn(1024, 1)
    x = (slope * pt.linspace(0, 1, 16) + 0.3 * pt.randn(1024, 16)).unsqueeze(-1)
    y = (slope[:, 0] > 0).long()
    m = CellNet("gru", 1, 24, 2).to(a.device)
    opt = pt.optim.RMSprop(m.parameters(), lr=0.005)
    for _ in range(a.steps(150)):
        opt.zero_grad()
        nn.functional.cross_entropy(m(x.to(a.device)), y.to(a.device)).backward()
        opt.step()
    acc = accuracy(m, x, y, a.device)
    return "accuracy", acc, acc > 0.85


def wide_mnist_roundtrip(a):
    """784 -> 1024 -> 10 trained, saved in the PTOR container and as a PyTorch checkpoint, loaded into fresh models: same accuracy."""
    x, y = mnist_like(a.samples, 7)
    xt, yt = mnist_like(2000, 8)

    def make():
        return nn.Sequential(nn.Linear(784, 1024), nn.ReLU(), nn.Linear(1024, 10)).to(a.device)
    m = make()
    fit_classifier(m, pt.optim.Adam(m.parameters(), lr=1e-3), x, y, a.epochs, 128, a.device)
    before = accuracy(m, xt, yt, a.device)
    with tempfile.TemporaryDirectory() as d:
        pt.save(m.state_dict(), os.path.join(d, "wide.ptor"))
        pt.save_pytorch(m.state_dict(), os.path.join(d, "wide.pt"))
        m2, m3 = make(), make()
        m2.load_state_dict(pt.load(os.path.join(d, "wide.ptor")))
        m3.load_state_dict(pt.load_pytorch(os.path.join(d, "wide.pt")))
    after, after_pt = accuracy(m2, xt, yt, a.device), accuracy(m3, xt, yt, a.device)
    return "accuracy before / after load", before, before > 0.9 and after == before and after_pt == before


TASKS = [("Linear regression", linear_regression), ("Logistic regression", logistic_regression), ("MLP on XOR", xor_mlp),
         ("Simple MNIST MLP", simple_mnist), ("Deep MNIST MLP", deep_mnist), ("MNIST with dropout", dropout_mnist), ("RNN sine wave", rnn_sine),
         ("LSTM sequence classifier", lstm_sequence), ("GRU trend detector", gru_trend), ("Wide MNIST + save / load", wide_mnist_roundtrip)]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="fewer samples and one epoch (a smoke run)")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--only", type=int, default=0, help="run only task N (1-10)")
    a = ap.parse_args(argv)
    a.samples, a.epochs = (4000, 1) if a.quick else (20000, 2)
    a.steps = lambda n: n                                    # the small tasks are quick either way
    failures = 0
    for i, (name, fn) in enumerate(TASKS, 1):
        if a.only and a.only != i:
            continue
        pt.manual_seed(100 + i)
        metric, value, ok = fn(a)
        print(f"[{i:2d}] {name:28s} {metric}: {value:.4f}  {'PASS' if ok else 'FAIL'}", flush=True)
        failures += not ok
    return failures


if __name__ == "__main__":
    sys.exit(main())
