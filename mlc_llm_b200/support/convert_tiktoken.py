"""tiktoken vocabulary -> HuggingFace ``tokenizer.json`` (plus ``vocab.json`` / ``merges.txt``).

Models such as Qwen (first generation) ship a ``*.tiktoken`` file: one ``<base64 token> <rank>`` pair per line,
ranks being both the token ids and the merge priorities. The runtime's tokenizer loader reads HuggingFace
files, so ``gen_config`` converts such a directory once. The reference does the same through the model's
remote tokenizer code (``python/mlc_llm/support/convert_tiktoken.py``); here the rank file is read directly,
no model code is executed.

A byte-pair vocabulary does not store its merges, but they follow from the ranks: a token of rank ``r`` is
the concatenation of the two pieces that remain when its bytes are merged using only ranks below ``r``.
"""

from __future__ import annotations

import base64
import json
import os
from typing import Dict, List, Optional, Tuple

# the split pattern of cl100k-style vocabularies (Qwen uses it unchanged)
DEFAULT_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                   r"\s*[\r\n]+|\s+(?!\S)|\s+")


def read_ranks(path: str) -> Dict[bytes, int]:
    ranks: Dict[bytes, int] = {}
    with open(path, "rb") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            token, rank = line.split()
            ranks[base64.b64decode(token)] = int(rank)
    return ranks


def _byte_alphabet() -> Dict[int, str]:
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    chars = keep[:]
    extra = 0
    for b in range(256):
        if b not in keep:
            keep.append(b)
            chars.append(256 + extra)
            extra += 1
    return {b: chr(c) for b, c in zip(keep, chars)}


def split_by_lower_ranks(token: bytes, ranks: Dict[bytes, int]) -> List[bytes]:
    """The pieces left when ``token``'s bytes are merged, lowest rank first, with ranks below its own."""
    limit = ranks[token]
    pieces = [token[i: i + 1] for i in range(len(token))]
    while len(pieces) > 1:
        best_at, best_rank = -1, limit
        for i in range(len(pieces) - 1):
            r = ranks.get(pieces[i] + pieces[i + 1])
            if r is not None and r < best_rank:
                best_at, best_rank = i, r
        if best_at < 0:
            break
        pieces[best_at: best_at + 2] = [pieces[best_at] + pieces[best_at + 1]]
    return pieces


def vocab_and_merges(ranks: Dict[bytes, int]) -> Tuple[Dict[str, int], List[str]]:
    alphabet = _byte_alphabet()

    def spell(raw: bytes) -> str:
        return "".join(alphabet[b] for b in raw)

    vocab = {spell(tok): rank for tok, rank in ranks.items()}
    merges: List[Tuple[int, str]] = []
    for tok, rank in ranks.items():
        if len(tok) < 2:
            continue
        parts = split_by_lower_ranks(tok, ranks)
        if len(parts) != 2:
            raise ValueError(f"token of rank {rank} does not split into two lower-ranked pieces ({len(parts)})")
        merges.append((rank, f"{spell(parts[0])} {spell(parts[1])}"))
    merges.sort()
    return vocab, [m for _, m in merges]


def convert_tiktoken(model_path: str, output_dir: Optional[str] = None, pattern: str = DEFAULT_PATTERN,
                     special_tokens: Optional[Dict[str, int]] = None) -> str:
    """Write ``tokenizer.json``, ``vocab.json`` and ``merges.txt`` for the ``*.tiktoken`` file under
    ``model_path``. Special tokens come from ``special_tokens`` or, if absent, from a
    ``special_tokens.json`` (``{token: id}``) beside the rank file. Returns the path of ``tokenizer.json``."""
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers  # pylint: disable=import-outside-toplevel
    from tokenizers import AddedToken  # pylint: disable=import-outside-toplevel

    output_dir = output_dir or model_path
    rank_files = [f for f in sorted(os.listdir(model_path)) if f.endswith(".tiktoken")]
    if not rank_files:
        raise FileNotFoundError(f"no *.tiktoken file under {model_path}")
    ranks = read_ranks(os.path.join(model_path, rank_files[0]))
    vocab, merges = vocab_and_merges(ranks)
    if special_tokens is None:
        side = os.path.join(model_path, "special_tokens.json")
        special_tokens = {}
        if os.path.exists(side):
            with open(side, encoding="utf-8") as f:
                special_tokens = {str(k): int(v) for k, v in json.load(f).items()}
    os.makedirs(output_dir, exist_ok=True)
    with open(os.path.join(output_dir, "vocab.json"), "w", encoding="utf-8") as f:
        json.dump(vocab, f, ensure_ascii=False)
    with open(os.path.join(output_dir, "merges.txt"), "w", encoding="utf-8") as f:
        f.write("#version: 0.2\n" + "\n".join(merges) + "\n")
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[tuple(m.split(" ")) for m in merges], fuse_unk=False,
                               byte_fallback=False))
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(pattern), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    # special tokens keep their recorded ids: they must be added in id order, directly after the ranks
    next_id = len(vocab)
    for name, idx in sorted(special_tokens.items(), key=lambda kv: kv[1]):
        while next_id < idx:   # unused ids between the ranks and the special tokens
            tok.add_special_tokens([AddedToken(f"<|extra_{next_id}|>", special=True)])
            next_id += 1
        tok.add_special_tokens([AddedToken(name, special=True)])
        next_id = max(next_id, idx + 1)
    out = os.path.join(output_dir, "tokenizer.json")
    tok.save(out)
    return out
