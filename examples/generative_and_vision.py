#!/usr/bin/env python
"""Five more training programs with the promethorch API, one per example family of the reference that the other scripts
of this folder do not cover: a variational auto-encoder (examples/vae), a GAN (examples/gan), a CIFAR-style ResNet-20
(examples/cifar), a vision transformer (examples/vit) and a sequence-to-sequence transformer (examples/transformer).

    python examples/generative_and_vision.py {vae,gan,resnet,vit,transformer,all} [--steps N] [--device cpu|cuda]

No dataset ships with the package: images are class prototypes plus noise (10 classes, 1x28x28 or 3x32x32), the
sequence task is "reverse the input".  Every program prints the first and the last value of what it minimises and
returns them, so a caller (or the test suite) can check that training moves.
"""
import argparse
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import promethorch as pt  # noqa: E402

nn, F = pt.nn, pt.nn.functional


def images(n, channels, side, seed, noise=0.35):
    g = pt.Generator().manual_seed(99)
    protos = pt.rand(10, channels, side, side, generator=g)
    g2 = pt.Generator().manual_seed(seed)
    y = pt.randint(0, 10, (n,), generator=g2)
    return (protos[y] + noise * pt.randn(n, channels, side, side, generator=g2)).clamp(0, 1), y


# ------------------------------------------------------------------------------------------------------------ VAE
class VAE(nn.Module):
    def __init__(self, latent=16):
        super().__init__()
        self.enc = nn.Sequential(nn.Flatten(), nn.Linear(784, 256), nn.ReLU())
        self.mu, self.logvar = nn.Linear(256, latent), nn.Linear(256, latent)
        self.dec = nn.Sequential(nn.Linear(latent, 256), nn.ReLU(), nn.Linear(256, 784), nn.Sigmoid())

    def forward(self, x):
        h = self.enc(x)
        mu, logvar = self.mu(h), self.logvar(h)
        z = mu + pt.randn_like(mu) * (0.5 * logvar).exp()
        return self.dec(z), mu, logvar


def train_vae(steps, dev):
    x, _ = images(2048, 1, 28, 1)
    m = VAE().to(dev)
    opt = pt.optim.Adam(m.parameters(), lr=2e-3)
    hist = []
    for i in range(steps):
        xb = x[(i * 128) % 1920:(i * 128) % 1920 + 128].to(dev)
        rec, mu, logvar = m(xb)
        # negative ELBO per image: reconstruction + KL(q(z|x) || N(0, I))
        loss = (F.binary_cross_entropy(rec, xb.flatten(1), reduction="sum") - 0.5 * (1 + logvar - mu.pow(2) - logvar.exp()).sum()) / xb.shape[0]
        opt.zero_grad()
        loss.backward()
        opt.step()
        hist.append(loss.item())
    return hist[0], hist[-1]


# ------------------------------------------------------------------------------------------------------------ GAN
def train_gan(steps, dev):
    """Generator and discriminator MLPs on flattened images; returns the mean distance from a generated image to the nearest
    class prototype before and after (real images sit at about 5, an untrained generator at about 16)."""
    x, _ = images(2048, 1, 28, 2, noise=0.1)
    x = x.flatten(1) * 2 - 1
    g = pt.Generator().manual_seed(99)
    protos = (pt.rand(10, 1, 28, 28, generator=g).flatten(1) * 2 - 1).to(dev)
    G = nn.Sequential(nn.Linear(32, 256), nn.LeakyReLU(0.2), nn.Linear(256, 784), nn.Tanh()).to(dev)
    D = nn.Sequential(nn.Linear(784, 256), nn.LeakyReLU(0.2), nn.Linear(256, 1)).to(dev)
    og, od = pt.optim.Adam(G.parameters(), lr=1e-3, betas=(0.5, 0.999)), pt.optim.Adam(D.parameters(), lr=1e-3, betas=(0.5, 0.999))
    bce = nn.BCEWithLogitsLoss()

    def distance():
        with pt.no_grad():
            return pt.cdist(G(pt.randn(256, 32, device=dev)), protos).min(1).values.mean().item()
    first = distance()
    for i in range(steps):
        real = x[(i * 64) % 1984:(i * 64) % 1984 + 64].to(dev)
        fake = G(pt.randn(64, 32, device=dev))
        od.zero_grad()
        (bce(D(real), pt.ones(64, 1, device=dev)) + bce(D(fake.detach()), pt.zeros(64, 1, device=dev))).backward()
        od.step()
        og.zero_grad()
        bce(D(fake), pt.ones(64, 1, device=dev)).backward()            # the non-saturating generator loss
        og.step()
    return first, distance()


# ------------------------------------------------------------------------------------------------------------ ResNet-20
def train_resnet(steps, dev):
    x, y = images(512, 3, 32, 3)
    m = pt.vision.ResNet20(num_classes=10).to(dev)
    opt = pt.optim.SGD(m.parameters(), lr=0.05, momentum=0.9, weight_decay=5e-4, nesterov=True)
    sched = pt.optim.OneCycleLR(opt, max_lr=0.1, total_steps=steps)
    hist = []
    for i in range(steps):
        j = (i * 32) % 480
        loss = F.cross_entropy(m(x[j:j + 32].to(dev)), y[j:j + 32].to(dev))
        opt.zero_grad()
        loss.backward()
        opt.step()
        sched.step()
        hist.append(loss.item())
    return hist[0], sum(hist[-3:]) / 3


# ------------------------------------------------------------------------------------------------------------ ViT
class ViT(nn.Module):
    """Patches of 7x7 -> linear embedding + class token + learned positions -> pre-norm transformer encoder -> head."""

    def __init__(self, dim=64, depth=2, heads=4, patch=7, side=28, classes=10):
        super().__init__()
        self.patch, n = patch, (side // patch) ** 2
        self.embed = nn.Linear(patch * patch, dim)
        self.cls = nn.Parameter(pt.zeros(1, 1, dim))
        self.pos = nn.Parameter(pt.randn(1, n + 1, dim) * 0.02)
        layer = nn.TransformerEncoderLayer(dim, heads, dim * 2, dropout=0.0, activation="gelu", batch_first=True, norm_first=True)
        self.encoder = nn.TransformerEncoder(layer, depth)
        self.norm, self.head = nn.LayerNorm(dim), nn.Linear(dim, classes)

    def forward(self, x):                                               # [B, 1, 28, 28]
        p = self.patch
        t = x.unfold(2, p, p).unfold(3, p, p).reshape(x.shape[0], -1, p * p)
        t = pt.cat([self.cls.expand(x.shape[0], -1, -1), self.embed(t)], 1) + self.pos
        return self.head(self.norm(self.encoder(t)[:, 0]))


def train_vit(steps, dev):
    x, y = images(1024, 1, 28, 4)
    m = ViT().to(dev)
    opt = pt.optim.AdamW(m.parameters(), lr=1e-3, weight_decay=0.05)
    hist = []
    for i in range(steps):
        j = (i * 64) % 960
        loss = F.cross_entropy(m(x[j:j + 64].to(dev)), y[j:j + 64].to(dev))
        opt.zero_grad()
        loss.backward()
        pt.nn.utils.clip_grad_norm_(m.parameters(), 1.0)
        opt.step()
        hist.append(loss.item())
    return hist[0], sum(hist[-3:]) / 3


# ------------------------------------------------------------------------------------------------------------ seq2seq transformer
class Reverser(nn.Module):
    """Encoder-decoder transformer that learns to emit its input reversed."""

    def __init__(self, vocab=20, dim=64):
        super().__init__()
        self.emb = nn.Embedding(vocab + 1, dim)                        # id `vocab` starts the output
        self.pos = nn.PositionalEncoding(dim, dropout=0.0, max_len=64, batch_first=True)
        self.tf = nn.Transformer(dim, 4, 2, 2, dim * 2, dropout=0.0, batch_first=True)
        self.out = nn.Linear(dim, vocab)
        self.scale = math.sqrt(dim)

    def forward(self, src, tgt_in):
        mask = nn.Transformer.generate_square_subsequent_mask(tgt_in.shape[1]).to(src.device)
        h = self.tf(self.pos(self.emb(src) * self.scale), self.pos(self.emb(tgt_in) * self.scale), tgt_mask=mask)
        return self.out(h)


def train_transformer(steps, dev):
    vocab, T = 20, 8
    m = Reverser(vocab).to(dev)
    opt = pt.optim.Adam(m.parameters(), lr=2e-3)
    sched = pt.optim.WarmupCosineAnnealingLR(opt, max(1, steps // 10), steps) if hasattr(pt.optim, "WarmupCosineAnnealingLR") else None
    hist = []
    for _ in range(steps):
        src = pt.randint(0, vocab, (64, T))
        tgt = src.flip(1)
        tgt_in = pt.cat([pt.full((64, 1), vocab), tgt[:, :-1]], 1)
        loss = F.cross_entropy(m(src.to(dev), tgt_in.to(dev)).reshape(-1, vocab), tgt.reshape(-1).to(dev))
        opt.zero_grad()
        loss.backward()
        opt.step()
        if sched is not None:
            sched.step()
        hist.append(loss.item())
    return hist[0], sum(hist[-3:]) / 3


PROGRAMS = {"vae": (train_vae, 60, "negative ELBO per image"), "gan": (train_gan, 300, "distance from a generated image to the nearest class prototype"),
            "resnet": (train_resnet, 30, "cross entropy"), "vit": (train_vit, 60, "cross entropy"), "transformer": (train_transformer, 150, "cross entropy")}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("which", choices=list(PROGRAMS) + ["all"])
    ap.add_argument("--steps", type=int, default=0, help="training steps (default: a short run per program)")
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    out = {}
    for name in (PROGRAMS if a.which == "all" else [a.which]):
        fn, steps, what = PROGRAMS[name]
        pt.manual_seed(7)
        first, last = fn(a.steps or steps, a.device)
        print(f"{name:12s} {what}: {first:.4f} -> {last:.4f}", flush=True)
        out[name] = (first, last)
    return out


if __name__ == "__main__":
    main()
