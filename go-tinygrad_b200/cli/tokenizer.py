"""A minimal reader of HF ``tokenizer.json`` byte-pair vocabularies, enough for
the command line's ``-prompt`` option.  Token ids are the library's real
interface; this sits outside the path from tokens to the next token.

Behaviour follows the reference's small tokenizer (loader/tokenizer/
tokenizer.go:92-188): the text is split at whitespace, every word but the first
gets the vocabulary's space marker in front ("Ġ" for byte-level vocabularies,
"▁" for SentencePiece ones), a word found whole in the vocabulary is one token,
otherwise its characters are merged by rank; decoding joins the pieces and
undoes the marker and the byte-to-character table.
"""
from __future__ import annotations

import json
from typing import Dict, List, Tuple


def _byte_table() -> Dict[str, int]:
    """The GPT-2 table from printable stand-in characters back to bytes."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[chr(b)] = b
        else:
            table[chr(256 + extra)] = b
            extra += 1
    return table


class Tokenizer:
    def __init__(self, path: str):
        with open(path, encoding="utf-8") as f:
            doc = json.load(f)
        model = doc.get("model", {})
        self.vocab: Dict[str, int] = dict(model.get("vocab", {}))
        for tok in doc.get("added_tokens", []):
            self.vocab.setdefault(tok["content"], tok["id"])
        self.rank: Dict[Tuple[str, str], int] = {}
        for i, m in enumerate(model.get("merges", [])):
            pair = tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m)
            if len(pair) == 2:
                self.rank[pair] = i
        self.pieces = {i: t for t, i in self.vocab.items()}
        # byte-level marker unless the vocabulary is a SentencePiece one (the reference's
        # own test: does it hold "▁the"; loader/tokenizer/tokenizer.go:99-102)
        self.marker = "▁" if "▁the" in self.vocab else "Ġ"
        self._bytes = _byte_table()

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for i, word in enumerate(text.split()):
            piece = word if i == 0 else self.marker + word
            if piece in self.vocab:
                ids.append(self.vocab[piece])
                continue
            parts = list(piece)
            while len(parts) > 1:
                best = min(range(len(parts) - 1),
                           key=lambda j: self.rank.get((parts[j], parts[j + 1]), len(self.rank)))
                if (parts[best], parts[best + 1]) not in self.rank:
                    break
                parts[best:best + 2] = [parts[best] + parts[best + 1]]
            ids.extend(self.vocab[p] for p in parts if p in self.vocab)
        return ids

    def decode(self, ids: List[int]) -> str:
        text = "".join(self.pieces.get(int(i), "") for i in ids).replace("▁", " ")
        raw = bytearray()
        for ch in text:
            if ch in self._bytes:
                raw.append(self._bytes[ch])
            else:
                raw.extend(ch.encode("utf-8"))
        return raw.decode("utf-8", errors="replace")
