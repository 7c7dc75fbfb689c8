"""Python handles of the native tokenizer glue.

``Tokenizer`` finds the tokenizer files of a model directory in the reference's search order
(``cpp/tokenizers/tokenizers.cc:143-195``): ``tokenizer.json`` (HuggingFace) -> ``tokenizer.model``
(SentencePiece) -> ``vocab.json`` + ``merges.txt`` (byte-level BPE) -> ``tokenizer_model`` (RWKV world
vocabulary, ``rwkv_world.py``).  Encoding is done by the HuggingFace / SentencePiece libraries (the world
vocabulary by a byte trie here); decoding, streaming detokenisation and stop-string matching
run in the native runtime from the post-processed token table.
"""

from __future__ import annotations

import json
import os
from typing import List, Optional, Sequence

from .. import _core


class Tokenizer:
    """Tokenizer bound to a model directory (or built synthetically for tests / benchmarks)."""

    def __init__(self, path: Optional[str] = None, *, _handle=None, _info=None):
        if _handle is not None:
            self._handle = _handle
            self._info = _info or json.loads(_handle.info_json())
            return
        if path is None:
            raise ValueError("a tokenizer path is required")
        self._handle, self._info = self._load(path)

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _load(path: str):
        directory = path if os.path.isdir(path) else os.path.dirname(path)
        tok_json = os.path.join(directory, "tokenizer.json")
        sp_model = os.path.join(directory, "tokenizer.model")
        if os.path.isfile(path) and path.endswith(".model"):
            sp_model, tok_json = path, ""
        if tok_json and os.path.exists(tok_json):
            from tokenizers import Tokenizer as HFTokenizer  # pylint: disable=import-outside-toplevel

            hf = HFTokenizer.from_file(tok_json)
            with open(tok_json, encoding="utf-8") as f:
                text = f.read()
            info = json.loads(_core.detect_tokenizer_info(text))
            size = hf.get_vocab_size(with_added_tokens=True)
            vocab = [""] * size
            for tok, idx in hf.get_vocab(with_added_tokens=True).items():
                if idx < size:
                    vocab[idx] = tok
            special = [int(t["id"]) for t in json.loads(text).get("added_tokens", [])
                       if t.get("special", False)]

            def encode(s: str):
                return hf.encode(s, add_special_tokens=False).ids

            return _core.Tokenizer(vocab, json.dumps(info), encode, special), info
        if os.path.exists(sp_model):
            import sentencepiece as spm  # pylint: disable=import-outside-toplevel

            sp = spm.SentencePieceProcessor(model_file=sp_model)
            vocab = [sp.id_to_piece(i) for i in range(sp.get_piece_size())]
            special = [i for i in range(sp.get_piece_size()) if sp.is_control(i)]
            info = {"token_postproc_method": "byte_fallback", "prepend_space_in_encode": True,
                    "strip_space_in_decode": True}
            return _core.Tokenizer(vocab, json.dumps(info), lambda s: sp.encode(s), special), info
        vocab_json = os.path.join(directory, "vocab.json")
        merges = os.path.join(directory, "merges.txt")
        if os.path.exists(vocab_json) and os.path.exists(merges):
            from tokenizers import Tokenizer as HFTokenizer  # pylint: disable=import-outside-toplevel
            from tokenizers import decoders, models, pre_tokenizers  # pylint: disable=import-outside-toplevel

            hf = HFTokenizer(models.BPE.from_file(vocab_json, merges))
            hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
            hf.decoder = decoders.ByteLevel()
            added = os.path.join(directory, "added_tokens.json")
            if os.path.exists(added):
                with open(added, encoding="utf-8") as f:
                    hf.add_special_tokens(list(json.load(f).keys()))
            size = hf.get_vocab_size(with_added_tokens=True)
            vocab = [""] * size
            for tok, idx in hf.get_vocab(with_added_tokens=True).items():
                vocab[idx] = tok
            info = {"token_postproc_method": "byte_level", "prepend_space_in_encode": False,
                    "strip_space_in_decode": False}
            return _core.Tokenizer(vocab, json.dumps(info),
                                   lambda s: hf.encode(s, add_special_tokens=False).ids, []), info
        world = os.path.join(directory, "tokenizer_model")
        if os.path.isfile(path) and os.path.basename(path) == "tokenizer_model":
            world = path
        if os.path.exists(world):
            from .rwkv_world import load_for_runtime  # pylint: disable=import-outside-toplevel

            vocab, info, encode, special = load_for_runtime(world)
            return _core.Tokenizer(vocab, json.dumps(info), encode, special), info
        raise ValueError(f"Cannot find any tokenizer under {path}")

    @staticmethod
    def synthetic(vocab_size: int) -> "Tokenizer":
        """Byte-level stand-in: ids 0..255 are the raw bytes, the rest print as ``<id>``. Used where
        no tokenizer files exist (random-weight benchmarks, unit tests)."""
        table = {}
        # GPT-2 byte <-> unicode map, forward direction
        bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
        cs = bs[:]
        n = 0
        for b in range(256):
            if b not in bs:
                bs.append(b)
                cs.append(256 + n)
                n += 1
        byte_to_char = {b: chr(c) for b, c in zip(bs, cs)}
        vocab = []
        for i in range(vocab_size):
            vocab.append(byte_to_char[i] if i < 256 else "".join(byte_to_char[b] for b in f"<{i}>".encode()))
            table[vocab[-1]] = i
        info = {"token_postproc_method": "byte_level", "prepend_space_in_encode": False,
                "strip_space_in_decode": False}

        def encode(s: str):
            return list(s.encode("utf-8"))

        return Tokenizer(_handle=_core.Tokenizer(vocab, json.dumps(info), encode, []), _info=info)

    # ------------------------------------------------------------------ API
    @property
    def handle(self):
        return self._handle

    @property
    def info(self) -> dict:
        return dict(self._info)

    def encode(self, text: str) -> List[int]:
        return list(self._handle.encode(text))

    def encode_batch(self, texts: Sequence[str]) -> List[List[int]]:
        return [self.encode(t) for t in texts]

    def decode(self, token_ids: Sequence[int]) -> str:
        return self._handle.decode(list(token_ids))

    def vocab_size(self) -> int:
        return self._handle.vocab_size()

    def id_to_token(self, token_id: int) -> str:
        return self._handle.id_to_token(token_id)

    def token_to_id(self, token: str) -> int:
        return self._handle.token_to_id(token)

    def post_processed_token_table(self) -> List[bytes]:
        return list(self._handle.post_processed_token_table())

    @staticmethod
    def detect_tokenizer_info(path: str) -> dict:
        tok_json = os.path.join(path, "tokenizer.json")
        if not os.path.exists(tok_json):
            return {"token_postproc_method": "byte_fallback", "prepend_space_in_encode": False,
                    "strip_space_in_decode": False}
        with open(tok_json, encoding="utf-8") as f:
            return json.loads(_core.detect_tokenizer_info(f.read()))


class TextStreamer:
    """Incremental detokeniser that never emits half a UTF-8 character."""

    def __init__(self, tokenizer: Tokenizer):
        self._impl = _core.TextStreamer(tokenizer.handle)

    def put(self, delta_tokens: Sequence[int]) -> str:
        return self._impl.put(list(delta_tokens))

    def finish(self) -> str:
        return self._impl.finish()


class StopStrHandler:
    """Token-stream filter that withholds text which may still grow into a stop string."""

    def __init__(self, stop_strs: Sequence[str], tokenizer: Tokenizer):
        self._impl = _core.StopStrHandler(list(stop_strs), tokenizer.handle)

    def put(self, token_id: int) -> List[int]:
        return list(self._impl.put(token_id))

    def finish(self) -> List[int]:
        return list(self._impl.finish())

    @property
    def stop_triggered(self) -> bool:
        return self._impl.stop_triggered


__all__ = ["Tokenizer", "TextStreamer", "StopStrHandler"]
