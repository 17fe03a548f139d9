"""Text <-> token ids for the command line, from a model folder's
``tokenizer.json``.

The reference prepares its vocabulary offline (convert.py:98-125: byte-level
vocabularies are mapped back from their printable stand-ins to raw bytes,
sentencepiece's U+2581 becomes a space) and encodes by greedy longest match
over a trie with a byte fallback (tokenizer.cpp:57-94); decoding strips the
space after BOS and maps <0xNN> tokens to bytes (tokenizer.cpp:44-55).  This
class does the same two steps at load time.  It is a convenience for prompts
given as text: every test and benchmark uses token ids.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional


def _byte_level_table() -> Dict[str, int]:
    """Printable stand-in character -> byte, the inverse of the byte-level
    vocabularies' encoding of raw bytes."""
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
    def __init__(self, pieces: List[bytes], bos_id: Optional[int], eos_ids: List[int]):
        self.pieces = pieces
        self.bos_id = bos_id
        self.eos_ids = list(eos_ids)
        self.byte_start = -1
        self.eot_id: Optional[int] = None
        self._index: Dict[bytes, int] = {}
        self._max_len = 1
        for i, p in enumerate(pieces):
            if p == b"<0x00>":
                self.byte_start = i
            elif p in (b"<|eot_id|>", b"<|end|>", b"<|im_end|>"):
                self.eot_id = i
            if p and p not in self._index:
                self._index[p] = i
                self._max_len = max(self._max_len, len(p))

    @classmethod
    def from_dir(cls, model_dir: str, vocab_size: int, bos_id: Optional[int],
                 eos_ids: List[int]) -> Optional["Tokenizer"]:
        path = os.path.join(model_dir, "tokenizer.json")
        if not os.path.isfile(path):
            return None
        with open(path, "r", encoding="utf-8") as f:
            tk = json.load(f)
        names = [""] * vocab_size
        for piece, idx in tk["model"]["vocab"].items():
            if idx < vocab_size:
                names[idx] = piece
        for added in tk.get("added_tokens", []):
            if added["id"] < vocab_size:
                names[added["id"]] = added["content"]
        byte_level = not tk["model"].get("byte_fallback", False)
        table = _byte_level_table()
        pieces = []
        for name in names:
            if byte_level:
                pieces.append(bytes(table.get(ch, 0) for ch in name))
            else:
                pieces.append(name.replace("▁", " ").encode("utf-8"))
        return cls(pieces, bos_id, eos_ids)

    @property
    def stop_ids(self) -> List[int]:
        return self.eos_ids + ([self.eot_id] if self.eot_id is not None else [])

    def encode(self, text: str, bos: bool = True) -> List[int]:
        data = text.encode("utf-8")
        out = [self.bos_id] if (bos and self.bos_id is not None) else []
        i = 0
        while i < len(data):
            hit = None
            for n in range(min(self._max_len, len(data) - i), 0, -1):
                tok = self._index.get(data[i:i + n])
                if tok is not None:
                    hit = (tok, n)
                    break
            if hit is None:
                if self.byte_start >= 0:
                    out.append(self.byte_start + data[i])
                i += 1
            else:
                out.append(hit[0])
                i += hit[1]
        return out

    def decode_one(self, prev: Optional[int], token: int) -> bytes:
        piece = self.pieces[token] if 0 <= token < len(self.pieces) else b""
        if prev is not None and prev == self.bos_id and piece[:1] == b" ":
            return piece[1:]
        if self.byte_start >= 0 and 0 <= token - self.byte_start < 256:
            return bytes([token - self.byte_start])
        return piece

    def decode(self, tokens: List[int], prev: Optional[int] = None) -> str:
        buf = b""
        for t in tokens:
            buf += self.decode_one(prev, t)
            prev = t
        return buf.decode("utf-8", errors="replace")
