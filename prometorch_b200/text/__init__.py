"""Text helpers: ``Vocab``, a trainable byte-pair encoder and a WordPiece tokenizer (torch/text/*.h)."""
from __future__ import annotations

from collections import Counter
from typing import Dict, Iterable, List, Tuple


class Vocab:
    def __init__(self, tokens: Iterable[str] = (), specials=("<pad>", "<unk>")):
        self.itos: List[str] = list(specials)
        self.stoi: Dict[str, int] = {t: i for i, t in enumerate(self.itos)}
        for t in tokens:
            self.add(t)
        self.unk = self.stoi.get("<unk>", 0)

    @classmethod
    def build(cls, texts: Iterable[str], min_freq: int = 1, specials=("<pad>", "<unk>")):
        c = Counter(w for t in texts for w in t.split())
        return cls([w for w, n in c.most_common() if n >= min_freq], specials)

    def add(self, t: str) -> int:
        if t not in self.stoi:
            self.stoi[t] = len(self.itos)
            self.itos.append(t)
        return self.stoi[t]

    def __len__(self):
        return len(self.itos)

    def encode(self, text: str) -> List[int]:
        return [self.stoi.get(w, self.unk) for w in text.split()]

    def decode(self, ids: Iterable[int]) -> str:
        return " ".join(self.itos[i] for i in ids)


class BPETokenizer:
    """Byte-pair encoding learned from a corpus; words end with ``</w>``."""

    def __init__(self):
        self.merges: List[Tuple[str, str]] = []
        self.vocab: Dict[str, int] = {}

    def train(self, texts: Iterable[str], vocab_size: int = 1000):
        words = Counter(tuple(w) + ("</w>",) for t in texts for w in t.split())
        symbols = {s for w in words for s in w}
        while len(symbols) + len(self.merges) < vocab_size:
            pairs = Counter()
            for w, n in words.items():
                for a, b in zip(w, w[1:]):
                    pairs[(a, b)] += n
            if not pairs:
                break
            (a, b), _ = pairs.most_common(1)[0]
            self.merges.append((a, b))
            new = {}
            for w, n in words.items():
                out, i = [], 0
                while i < len(w):
                    if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                        out.append(a + b)
                        i += 2
                    else:
                        out.append(w[i])
                        i += 1
                new[tuple(out)] = new.get(tuple(out), 0) + n
            words = new
        toks = sorted(symbols | {a + b for a, b in self.merges})
        self.vocab = {t: i for i, t in enumerate(["<unk>"] + toks)}
        return self

    def _word(self, w: str) -> List[str]:
        s = list(w) + ["</w>"]
        for a, b in self.merges:
            i, out = 0, []
            while i < len(s):
                if i + 1 < len(s) and s[i] == a and s[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(s[i])
                    i += 1
            s = out
        return s

    def encode(self, text: str) -> List[int]:
        return [self.vocab.get(t, 0) for w in text.split() for t in self._word(w)]

    def decode(self, ids: Iterable[int]) -> str:
        inv = {i: t for t, i in self.vocab.items()}
        return "".join(inv.get(i, "") for i in ids).replace("</w>", " ").strip()


class WordPieceTokenizer:
    def __init__(self, vocab: Iterable[str], unk: str = "[UNK]", max_chars: int = 100):
        self.vocab = {t: i for i, t in enumerate(vocab)}
        self.unk, self.max_chars = unk, max_chars

    def tokenize(self, text: str) -> List[str]:
        out = []
        for w in text.split():
            if len(w) > self.max_chars:
                out.append(self.unk)
                continue
            i, pieces, bad = 0, [], False
            while i < len(w):
                j, cur = len(w), None
                while i < j:
                    sub = ("##" if i > 0 else "") + w[i:j]
                    if sub in self.vocab:
                        cur = sub
                        break
                    j -= 1
                if cur is None:
                    bad = True
                    break
                pieces.append(cur)
                i = j
            out += [self.unk] if bad else pieces
        return out

    def encode(self, text: str) -> List[int]:
        return [self.vocab.get(t, self.vocab.get(self.unk, 0)) for t in self.tokenize(text)]
