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


# ---------------------------------------------------------------------------------------------- more tokenizers (torch/text/tokenizers.h)
class BasicTokenizer:
    """Lower-cases (optionally), splits on white space and cuts punctuation off as tokens of its own."""

    def __init__(self, lowercase: bool = True):
        self.lowercase = lowercase

    def tokenize(self, text: str) -> List[str]:
        import re
        if self.lowercase:
            text = text.lower()
        return re.findall(r"\w+|[^\w\s]", text, re.UNICODE)


class CharTokenizer:
    """One id per character, learned from a corpus; id 0 is the unknown character."""

    def __init__(self, corpus: str = ""):
        self.itos: List[str] = ["<unk>"] + sorted(set(corpus))
        self.stoi: Dict[str, int] = {c: i for i, c in enumerate(self.itos)}

    def __len__(self):
        return len(self.itos)

    def tokenize(self, text: str) -> List[str]:
        return list(text)

    def encode(self, text: str) -> List[int]:
        return [self.stoi.get(c, 0) for c in text]

    def decode(self, ids: Iterable[int]) -> str:
        return "".join(self.itos[i] for i in ids if 0 < i < len(self.itos))


# ---------------------------------------------------------------------------------------------- datasets and batching (torch/text/text.h)
class TextFileDataset:
    """One sample per non-empty line of a text file; ``labels`` (optional) gives one label per line."""

    def __init__(self, path: str, labels=None, skip_empty: bool = True):
        with open(path, encoding="utf-8") as f:
            self.lines = [ln.rstrip("\n") for ln in f if ln.strip() or not skip_empty]
        self.labels = list(labels) if labels is not None else None

    def __len__(self):
        return len(self.lines)

    def __getitem__(self, i):
        return (self.lines[i], self.labels[i]) if self.labels is not None else self.lines[i]


class CSVDataset:
    """Rows of a delimited file as lists of strings; ``label_column`` (a name or an index) is split off as the target."""

    def __init__(self, path: str, label_column=None, delimiter: str = ",", has_header: bool = True):
        import csv
        with open(path, newline="", encoding="utf-8") as f:
            rows = list(csv.reader(f, delimiter=delimiter))
        self.header = rows.pop(0) if has_header and rows else None
        col = self.header.index(label_column) if isinstance(label_column, str) else label_column
        self.rows, self.labels = [], []
        for r in rows:
            if not r:
                continue
            if col is not None:
                self.labels.append(r[col])
                r = r[:col] + r[col + 1:]
            self.rows.append(r)

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return (self.rows[i], self.labels[i]) if self.labels else self.rows[i]


class JSONLDataset:
    """One JSON object per line; ``text_key`` / ``label_key`` pick fields, without them the whole record comes back."""

    def __init__(self, path: str, text_key: str = None, label_key: str = None):
        import json
        with open(path, encoding="utf-8") as f:
            self.records = [json.loads(ln) for ln in f if ln.strip()]
        self.text_key, self.label_key = text_key, label_key

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        r = self.records[i]
        if self.text_key is None:
            return r
        return (r[self.text_key], r[self.label_key]) if self.label_key is not None else r[self.text_key]


def pad_sequence(batch, padding_value: int = 0, batch_first: bool = True, max_len: int = None):
    """Lists of ids -> one ``[B, T]`` (or ``[T, B]``) int64 tensor, cut or padded to ``max_len`` (default: the longest)."""
    import torch
    T = max_len if max_len is not None else max((len(s) for s in batch), default=0)
    out = torch.full((len(batch), T), padding_value, dtype=torch.int64)
    for i, s in enumerate(batch):
        s = list(s)[:T]
        out[i, :len(s)] = torch.tensor(s, dtype=torch.int64)
    return out if batch_first else out.t().contiguous()


def sequence_lengths(batch):
    import torch
    return torch.tensor([len(s) for s in batch], dtype=torch.int64)


def padding_mask(batch, max_len: int = None):
    """``[B, T]`` bool, True where a position holds padding."""
    import torch
    lens = sequence_lengths(batch)
    T = max_len if max_len is not None else int(lens.max()) if len(batch) else 0
    return torch.arange(T)[None, :] >= lens.clamp(max=T)[:, None]


def pack_padded_sequence(padded, lengths, batch_first: bool = True, enforce_sorted: bool = False):
    import torch
    return torch.nn.utils.rnn.pack_padded_sequence(padded, torch.as_tensor(lengths).cpu(), batch_first=batch_first, enforce_sorted=enforce_sorted)
