"""Byte-level BPE tokenizer compatible with the reference's ``bpe.json``
(scirust-sciagent/src/bpe.rs): ``{"vocab": {token string: id}, "merges": ["left right new", ...]}``,
specials ``<pad>=0 <bos>=1 <eos>=2 <unk>=3``. Two vocab flavours are read: the reversible "v2"
byte-level scheme (byte b is the single character ``chr(b)`` for b < 128 and ``chr(256 + b - 128)``
otherwise, so any UTF-8 text round-trips) and the legacy scheme (non-UTF-8 bytes written ``<NNN>``).
``encode`` applies the merges as repeated left-to-right passes over the whole sequence - in each
pass every adjacent pair that has a merge rule is replaced - until a pass changes nothing, which
is the reference's historical behaviour (bpe.rs:357-397), not priority-ordered BPE.
``BpeTrainer`` is a deterministic trainer: most frequent pair first, ties broken by the smaller
(left, right) id pair."""
from __future__ import annotations

import json
from collections import Counter
from pathlib import Path

SPECIAL_TOKENS = (("<pad>", 0), ("<bos>", 1), ("<eos>", 2), ("<unk>", 3))


def byte_to_unit(b: int) -> str:
    return chr(b) if b < 128 else chr(256 + b - 128)


def unit_to_byte(c: str):
    u = ord(c)
    if u < 128:
        return u
    if 256 <= u < 384:
        return u - 256 + 128
    return None


def _legacy_byte_str(b: int) -> str:
    try:
        return bytes([b]).decode("utf-8")
    except UnicodeDecodeError:
        return f"<{b}>"


class BpeTokenizer:
    def __init__(self, vocab: dict, merges: list):
        self.vocab = dict(vocab)
        self.merges = [tuple(m) for m in merges]
        n = max(self.vocab.values()) + 1 if self.vocab else 0
        self.rev = [""] * n
        for s, i in self.vocab.items():
            self.rev[i] = s
        self.reversible = all(byte_to_unit(b) in self.vocab for b in range(256))
        unk = self.vocab.get("<unk>", 3)
        if self.reversible:
            self.byte_ids = [self.vocab[byte_to_unit(b)] for b in range(256)]
        else:
            self.byte_ids = [self.vocab.get(_legacy_byte_str(b), unk) for b in range(256)]
        self.merge_lookup = {}
        for l, r, new in self.merges:
            self.merge_lookup[(l, r)] = new  # a later duplicate rule wins

    # ---- io
    @staticmethod
    def load_json(path) -> "BpeTokenizer":
        return BpeTokenizer.from_json_str(Path(path).read_text(encoding="utf-8"))

    @staticmethod
    def from_json_str(s: str) -> "BpeTokenizer":
        try:
            d = json.loads(s)
            merges = []
            for m in d["merges"]:
                a, b, c = m.split() if isinstance(m, str) else m
                merges.append((int(a), int(b), int(c)))
            vocab = {str(k): int(v) for k, v in d["vocab"].items()}
        except (KeyError, ValueError, TypeError, json.JSONDecodeError) as e:
            raise ValueError(f"malformed tokenizer json: {e}") from None
        return BpeTokenizer(vocab, merges)

    def save_json(self, path) -> None:
        d = {"merges": [f"{a} {b} {c}" for a, b, c in self.merges],
             "vocab": {k: self.vocab[k] for k in sorted(self.vocab)}}
        Path(path).write_text(json.dumps(d, ensure_ascii=False), encoding="utf-8")

    # ---- api
    def vocab_size(self) -> int:
        return len(self.rev)

    def special_id(self, name: str) -> int:
        return self.vocab.get(name, dict(SPECIAL_TOKENS).get(name, 3))

    def encode(self, text: str) -> list:
        ids = [self.byte_ids[b] for b in text.encode("utf-8")]
        if not ids or not self.merge_lookup:
            return ids
        look = self.merge_lookup
        while True:
            out, merged, i, n = [], False, 0, len(ids)
            while i < n:
                if i + 1 < n and ids[i] != 0 and ids[i + 1] != 0:
                    new = look.get((ids[i], ids[i + 1]))
                    if new is not None:
                        out.append(new)
                        i += 2
                        merged = True
                        continue
                out.append(ids[i])
                i += 1
            if not merged:
                return ids
            ids = out

    def encode_with_special(self, text: str, prepend_bos: bool = False, append_eos: bool = False) -> list:
        ids = [self.special_id("<bos>")] if prepend_bos else []
        ids += self.encode(text)
        if append_eos:
            ids.append(self.special_id("<eos>"))
        return ids

    def decode(self, ids) -> str:
        if self.reversible:
            out = bytearray()
            for i in ids:
                if i < len(SPECIAL_TOKENS) or i >= len(self.rev):
                    continue
                for ch in self.rev[i]:
                    b = unit_to_byte(ch)
                    if b is not None:
                        out.append(b)
            return out.decode("utf-8", errors="replace")
        parts = []
        for i in ids:
            if 0 <= i < len(self.rev):
                s = self.rev[i]
                if not self._is_non_text(s):
                    parts.append(s)
        return "".join(parts)

    @staticmethod
    def _is_non_text(s: str) -> bool:
        if s in dict(SPECIAL_TOKENS):
            return True
        return len(s) >= 3 and s[0] == "<" and s[-1] == ">" and s[1:-1].isdigit()


class BpeTrainer:
    def __init__(self, vocab_size: int, min_frequency: int = 2):
        self.vocab_size, self.min_frequency = vocab_size, min_frequency

    def train(self, texts) -> BpeTokenizer:
        vocab = {name: i for name, i in SPECIAL_TOKENS}
        for b in range(256):
            vocab[byte_to_unit(b)] = len(vocab)
        byte_ids = [vocab[byte_to_unit(b)] for b in range(256)]
        strs = {i: s for s, i in vocab.items()}
        seqs = [[byte_ids[b] for b in t.encode("utf-8")] for t in texts]
        merges = []
        while len(vocab) < self.vocab_size:
            counts = Counter()
            for s in seqs:
                counts.update(zip(s, s[1:]))
            if not counts:
                break
            (l, r), c = min(counts.items(), key=lambda kv: (-kv[1], kv[0]))
            if c < self.min_frequency:
                break
            tok = strs[l] + strs[r]
            if tok in vocab:
                new = vocab[tok]
            else:
                new = len(vocab)
                vocab[tok] = new
                strs[new] = tok
            merges.append((l, r, new))
            for k, s in enumerate(seqs):
                out, i = [], 0
                while i < len(s):
                    if i + 1 < len(s) and s[i] == l and s[i + 1] == r:
                        out.append(new)
                        i += 2
                    else:
                        out.append(s[i])
                        i += 1
                seqs[k] = out
            if len(merges) > 4 * self.vocab_size:
                break
        return BpeTokenizer(vocab, merges)
