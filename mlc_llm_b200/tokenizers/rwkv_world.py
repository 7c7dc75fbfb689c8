"""RWKV "world" tokenizer: a fixed vocabulary of byte strings matched greedily, longest first.

The model directory holds it as ``tokenizer_model`` (the reference looks for that file last, after
``tokenizer.json``, ``tokenizer.model`` and ``vocab.json`` + ``merges.txt``: ``cpp/tokenizers/tokenizers.cc:148-192``).
One entry per line: ``<id> <python literal of a str or bytes> <length in bytes>``. Id 0 is the
end-of-text token and has no line.
"""

from __future__ import annotations

import ast
from typing import Callable, Dict, List, Tuple


class _Node:
    __slots__ = ("next", "token")

    def __init__(self):
        self.next: Dict[int, "_Node"] = {}
        self.token = -1


def parse_vocab(path: str) -> Dict[int, bytes]:
    """``{id: bytes}`` of a world vocabulary file; every line's declared length is checked."""
    table: Dict[int, bytes] = {}
    with open(path, encoding="utf-8") as f:
        for lineno, line in enumerate(f, 1):
            line = line.rstrip("\n")
            if not line.strip():
                continue
            first, last = line.index(" "), line.rindex(" ")
            idx, length = int(line[:first]), int(line[last + 1:])
            value = ast.literal_eval(line[first + 1: last])
            raw = value.encode("utf-8") if isinstance(value, str) else bytes(value)
            if len(raw) != length:
                raise ValueError(f"{path}:{lineno}: entry {idx} is {len(raw)} bytes, the line says {length}")
            table[idx] = raw
    return table


class RWKVWorldTokenizer:
    """Greedy longest-match over a byte trie."""

    def __init__(self, table: Dict[int, bytes]):
        self.table = dict(table)
        self.table.setdefault(0, b"")  # end of text
        self.root = _Node()
        for idx, raw in self.table.items():
            if not raw:
                continue
            node = self.root
            for b in raw:
                node = node.next.setdefault(b, _Node())
            node.token = idx
        self.vocab_size = max(self.table) + 1

    @classmethod
    def from_file(cls, path: str) -> "RWKVWorldTokenizer":
        return cls(parse_vocab(path))

    def encode_bytes(self, data: bytes) -> List[int]:
        out: List[int] = []
        i, n = 0, len(data)
        while i < n:
            node, j, best, best_end = self.root, i, -1, i
            while j < n:
                node = node.next.get(data[j])
                if node is None:
                    break
                j += 1
                if node.token >= 0:
                    best, best_end = node.token, j
            if best < 0:
                raise ValueError(f"byte {data[i]:#04x} at offset {i} is not in the vocabulary")
            out.append(best)
            i = best_end
        return out

    def encode(self, text: str) -> List[int]:
        return self.encode_bytes(text.encode("utf-8"))

    def decode_bytes(self, ids) -> bytes:
        return b"".join(self.table.get(int(i), b"") for i in ids)

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")


def _byte_to_char() -> Dict[int, str]:
    """The GPT-2 byte <-> printable-character map (the byte-level post-processing of the token table)."""
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


def load_for_runtime(path: str) -> Tuple[List[str], dict, Callable[[str], List[int]], List[int]]:
    """``(token table, tokenizer info, encode function, special ids)`` in the form the native tokenizer takes:
    tokens are spelled in the byte-level alphabet so that the runtime's detokeniser restores the exact bytes,
    including tokens that end in the middle of a UTF-8 sequence."""
    tok = RWKVWorldTokenizer.from_file(path)
    b2c = _byte_to_char()
    vocab = ["".join(b2c[b] for b in tok.table.get(i, b"")) for i in range(tok.vocab_size)]
    info = {"token_postproc_method": "byte_level", "prepend_space_in_encode": False, "strip_space_in_decode": False}
    return vocab, info, tok.encode, [0]
