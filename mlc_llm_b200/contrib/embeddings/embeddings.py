"""Text embeddings from a locally loaded embedding model, with the method names retrieval libraries
expect.

Reference: ``python/mlc_llm/contrib/embeddings/embeddings.py`` (``MLCEmbeddings(model, model_lib, device)``
with ``embed(queries)``) and ``contrib/embeddings/openai.py`` (``embed_documents`` / ``embed_query``, the
interface of LangChain's embedding classes, without importing that library).
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from ...serve.embedding_engine import AsyncEmbeddingEngine


class MLCEmbeddings:
    """``embed`` returns an ``[n, dim]`` float32 array; ``embed_documents`` / ``embed_query`` return lists.
    Inputs are cut into batches of ``chunk_size`` texts; ``dimensions`` truncates and re-normalises each
    vector (Matryoshka-style)."""

    def __init__(self, model: str, model_lib: Optional[str] = None, device: str = "auto", *,
                 chunk_size: int = 64, dimensions: Optional[int] = None, **engine_kwargs):
        self.engine = AsyncEmbeddingEngine(model, model_lib, device, **engine_kwargs)
        self.chunk_size = max(1, int(chunk_size))
        self.dimensions = dimensions

    def embed(self, queries: Sequence[str]) -> np.ndarray:
        rows: List[List[float]] = []
        for i in range(0, len(queries), self.chunk_size):
            vectors, _ = self.engine.embed(list(queries[i: i + self.chunk_size]))
            rows.extend(vectors)
        if self.dimensions:
            rows = [self.engine.truncate(v, self.dimensions) for v in rows]
        return np.asarray(rows, dtype=np.float32).reshape(len(queries), -1)

    def embed_documents(self, texts: Sequence[str]) -> List[List[float]]:
        return self.embed(texts).tolist()

    def embed_query(self, text: str) -> List[float]:
        return self.embed([text])[0].tolist()

    def terminate(self) -> None:
        self.engine.terminate()
