"""RWKV world vocabulary and tiktoken conversion."""
import base64
import json

import pytest

from mlc_llm_b200.support.convert_tiktoken import convert_tiktoken, read_ranks, vocab_and_merges
from mlc_llm_b200.tokenizers import TextStreamer, Tokenizer
from mlc_llm_b200.tokenizers.rwkv_world import RWKVWorldTokenizer, parse_vocab


def _world_file(tmp_path):
    entries = [bytes([b]) for b in range(256)]
    entries += [b"he", b"hel", b"hello", b" wor", b" world", "é".encode(), "日本".encode(), "日".encode(),
                b"\xe6\x97"]  # the last one ends inside a UTF-8 sequence
    lines = []
    for i, raw in enumerate(entries, 1):
        try:
            lit = repr(raw.decode("utf-8")) if len(raw) > 1 or raw[0] < 128 else repr(raw)
        except UnicodeDecodeError:
            lit = repr(raw)
        lines.append(f"{i} {lit} {len(raw)}")
    path = tmp_path / "tokenizer_model"
    path.write_text("\n".join(lines) + "\n", encoding="utf-8")
    return path, entries


def test_world_vocabulary_is_matched_longest_first(tmp_path):
    path, entries = _world_file(tmp_path)
    table = parse_vocab(str(path))
    assert table[1] == b"\x00" and len(table) == len(entries)
    tok = RWKVWorldTokenizer(table)
    ids = tok.encode("hello world hey")
    assert [table[i] for i in ids][:2] == [b"hello", b" world"]
    assert tok.decode(ids) == "hello world hey"
    text = "日本 日 é\n"
    assert tok.decode(tok.encode(text)) == text
    assert [table[i] for i in tok.encode("日本")] == ["日本".encode()]


def test_world_vocabulary_through_the_runtime_tokenizer(tmp_path):
    path, _ = _world_file(tmp_path)
    tok = Tokenizer(str(tmp_path))
    text = "hello world 日本 é"
    ids = tok.encode(text)
    assert tok.decode(ids) == text
    # streaming detokenisation holds back a token that stops inside a character
    streamer = TextStreamer(tok)
    pieces = [streamer.put([i]) for i in ids] + [streamer.finish()]
    assert "".join(pieces) == text


def test_bad_length_is_reported(tmp_path):
    bad = tmp_path / "tokenizer_model"
    bad.write_text("1 'ab' 3\n")
    with pytest.raises(ValueError, match="the line says 3"):
        parse_vocab(str(bad))


def _tiktoken_dir(tmp_path):
    # a tiny byte-pair vocabulary built by actually running merges on a corpus
    corpus = "the theme of the thesis is the theory of them all there and then"
    words = [w.encode() for w in corpus.split(" ")]
    words = [b" " + w if i else w for i, w in enumerate(words)]
    ranks = {bytes([b]): b for b in range(256)}
    seqs = [[bytes([b]) for b in w] for w in words]
    while len(ranks) < 256 + 12:
        counts = {}
        for s in seqs:
            for a, b in zip(s[:-1], s[1:]):
                counts[(a, b)] = counts.get((a, b), 0) + 1
        (a, b), _ = max(counts.items(), key=lambda kv: (kv[1], kv[0]))
        ranks[a + b] = len(ranks)
        for s in seqs:
            i = 0
            while i < len(s) - 1:
                if s[i] == a and s[i + 1] == b:
                    s[i: i + 2] = [a + b]
                else:
                    i += 1
    d = tmp_path / "tk"
    d.mkdir()
    (d / "model.tiktoken").write_bytes(b"".join(base64.b64encode(t) + b" " + str(r).encode() + b"\n"
                                                for t, r in ranks.items()))
    (d / "special_tokens.json").write_text(json.dumps({"<|endoftext|>": len(ranks), "<|im_start|>": len(ranks) + 1}))
    return d, ranks, corpus, seqs


def test_tiktoken_ranks_become_a_huggingface_tokenizer(tmp_path):
    d, ranks, corpus, seqs = _tiktoken_dir(tmp_path)
    assert read_ranks(str(d / "model.tiktoken")) == ranks
    vocab, merges = vocab_and_merges(ranks)
    assert len(vocab) == len(ranks) and len(merges) == len(ranks) - 256
    out = convert_tiktoken(str(d))
    from tokenizers import Tokenizer as HF

    hf = HF.from_file(out)
    enc = hf.encode(corpus, add_special_tokens=False)
    # the ids are the ranks, and the segmentation is the one the merges produced when the vocabulary was built
    want = [ranks[p] for s in seqs for p in s]
    assert enc.ids == want
    assert hf.decode(enc.ids) == corpus
    assert hf.token_to_id("<|endoftext|>") == len(ranks) and hf.token_to_id("<|im_start|>") == len(ranks) + 1
    # and the runtime loader picks the converted files up
    tok = Tokenizer(str(d))
    assert tok.decode(tok.encode(corpus)) == corpus
