"""Embedding engine: BERT encoder against ``transformers``; decoder-style last-token pooling."""
import asyncio

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")
tokenizers = pytest.importorskip("tokenizers")

from mlc_llm_b200.serve.embedding_engine import AsyncEmbeddingEngine  # noqa: E402


@pytest.fixture(scope="module")
def bert_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("bert")
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + [chr(c) for c in range(97, 123)] + \
            ["##" + chr(c) for c in range(97, 123)] + ["hello", "world", "fast", "gpu", "##s"]
    tok = tokenizers.Tokenizer(tokenizers.models.WordPiece({t: i for i, t in enumerate(vocab)}, unk_token="[UNK]"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.Whitespace()
    tok.decoder = tokenizers.decoders.WordPiece()
    tok.save(str(d / "tokenizer.json"))
    import json
    json.dump({"cls_token": "[CLS]", "sep_token": "[SEP]", "pad_token": "[PAD]"}, open(d / "tokenizer_config.json", "w"))
    torch.manual_seed(0)
    cfg = transformers.BertConfig(vocab_size=len(vocab), hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                  intermediate_size=128, max_position_embeddings=64)
    model = transformers.BertModel(cfg, add_pooling_layer=False).float().eval()
    model.save_pretrained(d, safe_serialization=True)
    return str(d), model, tok


def test_bert_embeddings_match_transformers(bert_dir):
    path, hf, tok = bert_dir
    eng = AsyncEmbeddingEngine(path, device="cpu")
    texts = ["hello world", "fast gpus", "a b c d e f"]
    vecs, ntok = asyncio.run(eng.async_embed(texts))
    assert eng.model_type == "encoder" and eng.pooling_strategy == "cls" and len(vecs) == 3
    for text, v in zip(texts, vecs):
        ids = [2] + tok.encode(text).ids + [3]
        with torch.no_grad():
            h = hf(torch.tensor([ids])).last_hidden_state[0, 0]
        want = torch.nn.functional.normalize(h, dim=-1)
        assert torch.allclose(torch.tensor(v), want, atol=2e-4)
    mean_eng = AsyncEmbeddingEngine(path, device="cpu", pooling_strategy="mean", normalize=False)
    v2, _ = mean_eng.embed_sync(["hello world", "a"])
    ids = [2] + tok.encode("hello world").ids + [3]
    with torch.no_grad():
        want = hf(torch.tensor([ids])).last_hidden_state[0].mean(0)
    assert torch.allclose(torch.tensor(v2[0]), want, atol=2e-4)  # padding of the shorter input is masked out
    assert ntok > 0
    assert abs(sum(x * x for x in AsyncEmbeddingEngine.truncate(vecs[0], 16)) - 1.0) < 1e-5
    eng.terminate()
    mean_eng.terminate()


def test_decoder_embeddings_last_token_pooling():
    eng = AsyncEmbeddingEngine("random://tiny-llama?quant=q0f32&seed=4", device="cpu")
    assert eng.model_type == "decoder" and eng.pooling_strategy == "last"
    a, _ = eng.embed_sync([[5, 6, 7, 8], [9, 10]])
    b, _ = eng.embed_sync([[9, 10]])
    assert len(a) == 2 and len(a[0]) == 256
    assert torch.allclose(torch.tensor(a[1]), torch.tensor(b[0]), atol=1e-5)  # batching does not change a vector
    assert abs(sum(x * x for x in a[0]) - 1.0) < 1e-4
    eng.terminate()


def test_contrib_embeddings_wrapper(bert_dir):
    from mlc_llm_b200.contrib.embeddings import MLCEmbeddings

    path, _, _ = bert_dir
    emb = MLCEmbeddings(path, device="cpu", chunk_size=2)
    try:
        texts = ["hello world", "fast gpus", "a b c d e f"]
        mat = emb.embed(texts)
        assert mat.shape == (3, 64) and np.allclose(np.linalg.norm(mat, axis=1), 1.0, atol=1e-4)
        direct, _ = emb.engine.embed(texts)
        assert np.allclose(mat, np.asarray(direct), atol=1e-6)       # batching does not change the vectors
        assert np.allclose(emb.embed_query("fast gpus"), mat[1], atol=1e-5)
        assert len(emb.embed_documents(texts)) == 3
        emb.dimensions = 16
        small = emb.embed(texts)
        assert small.shape == (3, 16) and np.allclose(np.linalg.norm(small, axis=1), 1.0, atol=1e-4)
    finally:
        emb.terminate()


def test_embeddings_over_rest(bert_dir):
    """``/v1/embeddings`` of a server started with ``--embedding-model``: float and base64 encodings, the
    ``dimensions`` truncation (re-normalised), token usage; the vectors are those of the engine called directly
    (reference: ``tests/python/serve/server/test_embedding_server.py``)."""
    import base64
    import socket
    import struct

    import requests

    from mlc_llm_b200.serve.server import PopenServer

    path, _hf, _tok = bert_dir
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    srv = PopenServer("random://tiny-llama?quant=q0f32&seed=3", "cpu", mode="local", port=port, embedding_model=path)
    srv.start(timeout=240)
    try:
        texts = ["hello world", "fast gpus"]
        r = requests.post(srv.base_url + "/v1/embeddings", json={"model": path, "input": texts}, timeout=60)
        assert r.status_code == 200, r.text
        body = r.json()
        vecs = [np.asarray(d["embedding"], dtype=np.float32) for d in body["data"]]
        assert [d["index"] for d in body["data"]] == [0, 1] and body["usage"]["prompt_tokens"] > 0
        eng = AsyncEmbeddingEngine(path, device="cpu")
        want, n_tok = asyncio.run(eng.async_embed(texts))
        assert body["usage"]["prompt_tokens"] == n_tok
        for got, ref in zip(vecs, want):
            assert np.allclose(got, np.asarray(ref, dtype=np.float32), atol=1e-5)
            assert abs(float(np.linalg.norm(got)) - 1.0) < 1e-4
        r = requests.post(srv.base_url + "/v1/embeddings",
                          json={"model": path, "input": "hello world", "encoding_format": "base64", "dimensions": 16},
                          timeout=60)
        assert r.status_code == 200, r.text
        raw = base64.b64decode(r.json()["data"][0]["embedding"])
        short = np.asarray(struct.unpack(f"<{len(raw) // 4}f", raw), dtype=np.float32)
        assert short.shape == (16,) and abs(float(np.linalg.norm(short)) - 1.0) < 1e-4
        head = vecs[0][:16] / np.linalg.norm(vecs[0][:16])
        assert np.allclose(short, head, atol=1e-5)
    finally:
        srv.terminate()
