#!/usr/bin/env python
"""Character-level GPT on a text file (the counterpart of examples/shakespeare in the reference).

    python examples/shakespeare_gpt.py [--text FILE] [--iters 300] [--device cuda|cpu]

6 layers, d_model 384, 6 heads, context 256, weight-tied embedding: the network of the DDP training benchmark.  On a
GPU the blocks run on the package's fused kernels (FlashAttention, fused LayerNorm/GELU MLP, fused AdamW); without
``--text`` a short built-in passage is repeated so that the script runs anywhere.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import promethorch as pt  # noqa: E402
from prometorch_b200.models.gpt import CharGPT, GPTConfig  # noqa: E402

BUILTIN = ("To be, or not to be, that is the question:\nWhether 'tis nobler in the mind to suffer\n"
           "The slings and arrows of outrageous fortune,\nOr to take arms against a sea of troubles\nAnd by opposing end them.\n") * 200


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--text", default=None)
    ap.add_argument("--iters", type=int, default=300)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--device", default="cuda" if pt.cuda_is_available() else "cpu")
    ap.add_argument("--layers", type=int, default=6)
    a = ap.parse_args()
    text = open(a.text, encoding="utf-8").read() if a.text else BUILTIN
    chars = sorted(set(text))
    stoi = {c: i for i, c in enumerate(chars)}
    data = pt.tensor([stoi[c] for c in text], dtype=pt.int64)
    cfg = GPTConfig(vocab_size=max(len(chars), 2), n_layer=a.layers)
    model = CharGPT(cfg).to(a.device)
    if a.device != "cpu":
        model = model.to(pt.bfloat16)
    opt = pt.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    sched = pt.optim.WarmupCosineAnnealingLR(opt, warmup_epochs=20, total_epochs=a.iters)
    T = cfg.block_size
    for it in range(a.iters):
        ix = pt.randint(0, len(data) - T - 1, (a.batch,))
        x = pt.stack([data[i:i + T] for i in ix]).to(a.device)
        y = pt.stack([data[i + 1:i + T + 1] for i in ix]).to(a.device)
        opt.zero_grad()
        loss = model(x, y)
        loss.backward()
        pt.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        sched.step()
        if it % 50 == 0 or it == a.iters - 1:
            print(f"iter {it}: loss {float(loss):.3f}")
    # sample
    model.eval()
    ctx = data[:1].reshape(1, 1).to(a.device)
    with pt.no_grad():
        for _ in range(200):
            logits = model(ctx[:, -T:])
            nxt = pt.multinomial(pt.softmax(logits[:, -1].float(), -1), 1)
            ctx = pt.cat([ctx, nxt], 1)
    print("".join(chars[i] for i in ctx[0].tolist()))


if __name__ == "__main__":
    main()
