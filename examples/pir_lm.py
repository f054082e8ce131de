#!/usr/bin/env python
"""A small language model built on gated linear recurrences (the reference's PIR example, examples/pir):
each sub-layer computes h[t] = g[t] * h[t-1] + x[t] along the sequence with input-dependent gates, which on a GPU is
the chunked parallel scan of this package (``ops.scan.linear_scan``), forward and backward.

    python examples/pir_lm.py [--iters 200] [--device cuda|cpu]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import promethorch as pt  # noqa: E402
from prometorch_b200.ops.scan import linear_scan  # noqa: E402


class PIRLayer(pt.nn.Module):
    def __init__(self, d):
        super().__init__()
        self.norm = pt.nn.LayerNorm(d)
        self.inp = pt.nn.Linear(d, 2 * d)
        self.out = pt.nn.Linear(d, d)

    def forward(self, x):
        v, g = self.inp(self.norm(x)).chunk(2, -1)
        g = pt.sigmoid(g)
        return x + self.out(linear_scan(g.contiguous(), ((1 - g) * v).contiguous()))


class PIRLM(pt.nn.Module):
    def __init__(self, vocab, d=256, layers=4):
        super().__init__()
        self.emb = pt.nn.Embedding(vocab, d)
        self.layers = pt.nn.ModuleList([PIRLayer(d) for _ in range(layers)])
        self.head = pt.nn.Linear(d, vocab)

    def forward(self, idx):
        x = self.emb(idx)
        for l in self.layers:
            x = l(x)
        return self.head(x)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--device", default="cuda" if pt.cuda_is_available() else "cpu")
    a = ap.parse_args()
    pt.manual_seed(0)
    vocab, T, B = 64, 128, 16
    # a learnable synthetic language: every token is the sum (mod vocab) of the two before it, so predicting the next
    # one needs the state the recurrence carries
    data = pt.zeros(B * 64, T + 1, dtype=pt.int64)
    data[:, :2] = pt.randint(0, vocab, (B * 64, 2))
    for t in range(2, T + 1):
        data[:, t] = (data[:, t - 1] + data[:, t - 2]) % vocab
    model = PIRLM(vocab).to(a.device)
    opt = pt.optim.AdamW(model.parameters(), lr=2e-3)
    for it in range(a.iters):
        ix = pt.randint(0, data.shape[0], (B,))
        seq = data[ix].to(a.device)
        x, y = seq[:, :T], seq[:, 1:T + 1]
        opt.zero_grad()
        loss = pt.nn.functional.cross_entropy(model(x).reshape(-1, vocab), y.reshape(-1))
        loss.backward()
        opt.step()
        if it % 40 == 0 or it == a.iters - 1:
            print(f"iter {it}: loss {float(loss):.3f}")


if __name__ == "__main__":
    main()
