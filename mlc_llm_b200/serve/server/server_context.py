"""Registry of the engines one server process hosts (reference:
``python/mlc_llm/serve/server/server_context.py:12-72``)."""

from __future__ import annotations

from typing import Dict, List, Optional


class ServerContext:
    """Maps model names to running engines; one instance is current per process."""

    _current: Optional["ServerContext"] = None
    enable_debug: bool = False

    def __init__(self) -> None:
        self._engines: Dict[str, object] = {}
        self._embedding_engine = None
        self._embedding_model: Optional[str] = None
        self.api_key: Optional[str] = None

    def __enter__(self) -> "ServerContext":
        if ServerContext._current is not None:
            raise RuntimeError("a server context is already active in this process")
        ServerContext._current = self
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        for engine in self._engines.values():
            engine.terminate()
        if self._embedding_engine is not None:
            self._embedding_engine.terminate()
        self._engines.clear()
        self._embedding_engine = None
        ServerContext._current = None

    @staticmethod
    def current() -> Optional["ServerContext"]:
        return ServerContext._current

    def add_model(self, hosted_model: str, engine) -> None:
        if hosted_model in self._engines:
            raise RuntimeError(f"model {hosted_model!r} is already served")
        self._engines[hosted_model] = engine

    def set_embedding_engine(self, model: str, engine) -> None:
        self._embedding_model, self._embedding_engine = model, engine

    def get_engine(self, model: Optional[str]):
        """The engine serving ``model``; with a single hosted model any name resolves to it (the
        reference accepts requests that omit or misname the model in that case)."""
        if model in self._engines:
            return self._engines[model]
        if len(self._engines) == 1:
            return next(iter(self._engines.values()))
        return None

    def get_embedding_engine(self, model: Optional[str]):
        if self._embedding_engine is None:
            return None
        if model in (None, self._embedding_model) or self._embedding_engine is not None:
            return self._embedding_engine
        return None

    def get_model_list(self) -> List[str]:
        names = list(self._engines)
        if self._embedding_model is not None:
            names.append(self._embedding_model)
        return names
