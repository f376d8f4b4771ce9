"""Reader for the reference's one-file tokenizer (``tokenizer.json`` with ``vocab``, ``merges``
and ``special_tokens``, bytes mapped to latin-1 strings: src/scratch_llm/tokenizer.py:207-236)
and the byte-level BPE encoding it describes (:238-290): split out special tokens, cut the rest
with the GPT-2 pattern, and merge each piece's bytes in the order the merges were learned.

Only the command line uses it; the engine itself takes and returns token ids.
"""

from __future__ import annotations

import json
from pathlib import Path

import regex

_PIECES = regex.compile(
    r"""'(?:[sdmt]|ll|ve|re)| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""")


class Tokenizer:
    def __init__(self, vocab: dict[int, bytes], merges: list[tuple[bytes, bytes]],
                 special_tokens: list[str]) -> None:
        self.vocab = dict(vocab)
        self.special_tokens = list(special_tokens)
        self._id_of = {b: i for i, b in self.vocab.items()}
        self._rank = {pair: r for r, pair in enumerate(merges)}
        for s in self.special_tokens:
            b = s.encode("utf-8")
            if b not in self._id_of:
                new = max(self.vocab, default=-1) + 1
                self.vocab[new] = b
                self._id_of[b] = new
        self._special = {s: self._id_of[s.encode("utf-8")] for s in self.special_tokens}
        self._split = regex.compile("(" + "|".join(
            regex.escape(s) for s in sorted(self.special_tokens, key=len, reverse=True)) + ")") \
            if self.special_tokens else None

    @classmethod
    def load(cls, path: str | Path) -> "Tokenizer":
        raw = json.loads(Path(path).read_text(encoding="utf-8"))
        vocab = {int(i): s.encode("latin-1") for i, s in raw["vocab"].items()}
        merges = [(a.encode("latin-1"), b.encode("latin-1")) for a, b in raw["merges"]]
        return cls(vocab, merges, list(raw.get("special_tokens", [])))

    def _merge(self, piece: bytes) -> list[int]:
        parts = [bytes([b]) for b in piece]
        while len(parts) > 1:
            ranked = [(self._rank.get((parts[i], parts[i + 1]), 1 << 60), i)
                      for i in range(len(parts) - 1)]
            rank, i = min(ranked)
            if rank == 1 << 60:
                break
            parts[i:i + 2] = [parts[i] + parts[i + 1]]
        return [self._id_of[p] for p in parts]

    def encode(self, text: str) -> list[int]:
        ids: list[int] = []
        segments = self._split.split(text) if self._split else [text]
        for seg in segments:
            if not seg:
                continue
            if seg in self._special:
                ids.append(self._special[seg])
            else:
                for m in _PIECES.finditer(seg):
                    ids.extend(self._merge(m.group().encode("utf-8")))
        return ids

    def decode(self, ids) -> str:
        """The text of ``ids``; an id the vocabulary does not hold (a model whose output matrix
        is larger than its tokenizer) becomes the replacement character."""
        unknown = "\ufffd".encode("utf-8")
        return b"".join(self.vocab.get(i, unknown) for i in ids).decode("utf-8", errors="replace")
