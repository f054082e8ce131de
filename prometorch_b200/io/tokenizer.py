"""Tokenizer driven by GGUF metadata (``tokenizer.ggml.*``): SentencePiece-style BPE (``▁`` word
boundary, score-ordered merges, ``<0xNN>`` byte fallback) and GPT-2 byte-level BPE (regex
pre-tokeniser, merge ranks), with special tokens split out before either runs.  Counterpart of the
reference's GGUFTokenizer (torch/io/tokenizer.h:24-646)."""
from __future__ import annotations

import heapq
import re
from typing import Dict, Iterable, List, Optional, Tuple

try:
    import regex as _re
    _GPT2_PAT = _re.compile(r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""")
    # the pre-tokenisers newer byte-level vocabularies were trained with (the file names one in tokenizer.ggml.pre)
    _QWEN2_PAT = _re.compile(r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+""")
    _LLAMA3_PAT = _re.compile(r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+""")
except Exception:  # pragma: no cover
    _re = re
    _GPT2_PAT = re.compile(r"""'s|'t|'re|'ve|'m|'ll|'d| ?[A-Za-z]+| ?[0-9]+| ?[^\sA-Za-z0-9]+|\s+(?!\S)|\s+""")
    _QWEN2_PAT = _LLAMA3_PAT = _GPT2_PAT


def pretokenizer_pattern(pre: str):
    """The split pattern for a ``tokenizer.ggml.pre`` name: qwen2-style (single digits, one leading symbol joins a word,
    newlines close a run), llama-3-style (digits in groups of up to three), else GPT-2's."""
    pre = (pre or "").lower()
    if pre in ("qwen2", "qwen", "deepseek-r1-qwen", "qwen3"):
        return _QWEN2_PAT
    if pre in ("llama3", "llama-bpe", "llama-v3", "llama4", "smaug-bpe"):
        return _LLAMA3_PAT
    return _GPT2_PAT


def _bytes_to_unicode() -> Dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, [chr(c) for c in cs]))


_B2U = _bytes_to_unicode()
_U2B = {v: k for k, v in _B2U.items()}


class GGUFTokenizer:
    def __init__(self, tokens: List[str], model: str = "llama", scores: Optional[List[float]] = None,
                 merges: Optional[List[str]] = None, token_types: Optional[List[int]] = None, bos_id: int = -1, eos_id: int = -1,
                 add_bos: bool = False, pre: str = ""):
        self.tokens, self.model = list(tokens), model
        self.pre, self._pat = pre or "", pretokenizer_pattern(pre)
        self.vocab: Dict[str, int] = {t: i for i, t in enumerate(self.tokens)}
        self.scores = list(scores) if scores is not None else [0.0] * len(self.tokens)
        self.token_types = list(token_types) if token_types is not None else [1] * len(self.tokens)
        self.bos_id, self.eos_id, self.add_bos = bos_id, eos_id, add_bos
        self.ranks: Dict[Tuple[str, str], int] = {}
        for r, m in enumerate(merges or []):
            a, _, b = m.partition(" ")
            self.ranks[(a, b)] = r
        self.byte_ids = {b: self.vocab.get(f"<0x{b:02X}>", -1) for b in range(256)}
        specials = [t for i, t in enumerate(self.tokens) if self.token_types[i] in (3, 4) or (t.startswith("<|") and t.endswith("|>"))]
        specials = [s for s in specials if s]
        self._special_re = re.compile("(" + "|".join(re.escape(s) for s in sorted(specials, key=len, reverse=True)) + ")") if specials else None

    @classmethod
    def from_reader(cls, reader) -> "GGUFTokenizer":
        g = reader.get
        toks = g("tokenizer.ggml.tokens")
        if toks is None:
            raise ValueError("GGUF file carries no tokenizer")
        scores, types = g("tokenizer.ggml.scores"), g("tokenizer.ggml.token_type")
        return cls(list(toks), g("tokenizer.ggml.model", "llama"), None if scores is None else list(scores), g("tokenizer.ggml.merges"),
                   None if types is None else list(types), int(g("tokenizer.ggml.bos_token_id", -1)),
                   int(g("tokenizer.ggml.eos_token_id", -1)), bool(g("tokenizer.ggml.add_bos_token", False)), str(g("tokenizer.ggml.pre", "") or ""))

    @property
    def vocab_size(self) -> int:
        return len(self.tokens)

    # ------------------------------------------------------------------ encode
    def encode(self, text: str, add_bos: Optional[bool] = None, parse_special: bool = True) -> List[int]:
        ids: List[int] = []
        if (self.add_bos if add_bos is None else add_bos) and self.bos_id >= 0:
            ids.append(self.bos_id)
        parts = self._special_re.split(text) if (parse_special and self._special_re is not None) else [text]
        first = True
        for part in parts:
            if not part:
                continue
            if parse_special and part in self.vocab and self._special_re is not None and self._special_re.fullmatch(part):
                ids.append(self.vocab[part])
            elif self.model == "gpt2":
                ids.extend(self._encode_gpt2(part))
            else:
                ids.extend(self._encode_spm(part, first))
            first = False
        return ids

    def _encode_spm(self, text: str, prefix_space: bool) -> List[int]:
        text = text.replace(" ", "▁")
        if prefix_space and not text.startswith("▁"):
            text = "▁" + text
        if not text:
            return []
        # whole-word shortcut: a text made only of words that are vocabulary entries themselves needs no merging
        # (also reaches entries no merge chain leads to, like the reference's longest-match fallback, tokenizer.h:463)
        if text.startswith("▁"):
            ids = [self.vocab.get("▁" + w) for w in text[1:].split("▁")]
            if all(t is not None for t in ids):
                return ids
        syms = list(text)
        n = len(syms)
        prev, nxt, alive = list(range(-1, n - 1)), list(range(1, n + 1)), [True] * n
        heap = []

        def push(i):
            j = nxt[i]
            if j < n:
                tid = self.vocab.get(syms[i] + syms[j])
                if tid is not None:
                    heapq.heappush(heap, (-self.scores[tid], i, syms[i], syms[j]))
        for i in range(n - 1):
            push(i)
        while heap:
            _, i, a, b = heapq.heappop(heap)
            j = nxt[i]
            if not alive[i] or j >= n or not alive[j] or syms[i] != a or syms[j] != b:
                continue
            syms[i] = a + b
            alive[j] = False
            nxt[i] = nxt[j]
            if nxt[j] < n:
                prev[nxt[j]] = i
            if prev[i] >= 0:
                push(prev[i])
            push(i)
        out = []
        i = 0
        while i < n:
            if alive[i]:
                tid = self.vocab.get(syms[i])
                if tid is not None:
                    out.append(tid)
                else:
                    for bt in syms[i].encode("utf-8"):
                        out.append(self.byte_ids[bt] if self.byte_ids[bt] >= 0 else 0)
            i = nxt[i] if alive[i] else i + 1
        return out

    def _bpe(self, word: Tuple[str, ...]) -> Tuple[str, ...]:
        while len(word) > 1:
            best, bi = None, -1
            for i in range(len(word) - 1):
                r = self.ranks.get((word[i], word[i + 1]))
                if r is not None and (best is None or r < best):
                    best, bi = r, i
            if best is None:
                break
            word = word[:bi] + (word[bi] + word[bi + 1],) + word[bi + 2:]
        return word

    def _encode_gpt2(self, text: str) -> List[int]:
        out = []
        for piece in self._pat.findall(text):
            mapped = "".join(_B2U[b] for b in piece.encode("utf-8"))
            for tok in self._bpe(tuple(mapped)):
                tid = self.vocab.get(tok)
                if tid is not None:
                    out.append(tid)
                else:
                    out.extend(self.vocab.get(c, 0) for c in tok)
        return out

    # ------------------------------------------------------------------ decode
    def decode_token(self, tid: int) -> str:
        return self.decode([tid], strip_leading_space=False)

    def decode(self, ids: Iterable[int], skip_special: bool = True, strip_leading_space: bool = True) -> str:
        buf = bytearray()
        for tid in ids:
            if tid < 0 or tid >= len(self.tokens):
                continue
            if skip_special and (self.token_types[tid] == 3 or tid in (self.bos_id,)):
                continue
            t = self.tokens[tid]
            if self.model == "gpt2":
                buf.extend(bytes(_U2B.get(c, ord("?") if ord(c) > 255 else ord(c)) for c in t))
            elif len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
                buf.append(int(t[3:5], 16))
            else:
                buf.extend(t.replace("▁", " ").encode("utf-8"))
        s = buf.decode("utf-8", errors="replace")
        if self.model != "gpt2" and strip_leading_space and s.startswith(" "):
            s = s[1:]
        return s
