"""Embedding helpers (reference: ``python/mlc_llm/contrib/embeddings``)."""
from .embeddings import MLCEmbeddings

__all__ = ["MLCEmbeddings"]
