"""Python handle of the native JSON engine (reference: ``python/mlc_llm/json_ffi/engine.py:209-295``).

Requests go in as OpenAI chat-completion JSON strings; template rendering, tokenisation, scheduling
and detokenisation all happen in C++ (``csrc/serve/json_ffi_engine.cc``); chunks come back as JSON and
are validated into ``ChatCompletionStreamResponse`` objects here."""

from __future__ import annotations

import json
import queue
import threading
from typing import Any, Dict, Iterator, List, Literal, Optional, Union

import torch

from .. import _core
from ..protocol import openai_api_protocol as openai
from ..serve import engine_base
from ..serve.config import EngineConfig
from ..serve.engine_base import EngineRuntime


class _Completions:
    def __init__(self, engine: "JSONFFIEngine"):
        self._engine = engine

    def create(self, *, messages: List[Dict[str, Any]], model: Optional[str] = None, stream: bool = True,
               request_id: Optional[str] = None, **kwargs) -> Iterator[openai.ChatCompletionStreamResponse]:
        body = dict(kwargs, messages=messages, model=model or self._engine.model, stream=stream)
        rid = request_id or engine_base.create_request_id("chatcmpl", body.get("user"))
        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
        body.setdefault("stream_options", {"include_usage": True})  # the final chunk marks the end
        return self._engine._raw_chat_completion(json.dumps(body), include_usage, rid)  # pylint: disable=protected-access


class _Chat:
    def __init__(self, engine: "JSONFFIEngine"):
        self.completions = _Completions(engine)


class JSONFFIEngine:
    def __init__(self, model: str, device: Union[str, torch.device] = "auto", *, model_lib: Optional[str] = None,
                 mode: Literal["local", "interactive", "server"] = "local",
                 engine_config: Optional[EngineConfig] = None) -> None:
        engine_config = engine_config or EngineConfig()
        engine_config.model = model
        if model_lib is not None:
            engine_config.model_lib = model_lib
        engine_config.mode = engine_config.mode or mode
        self.model = model
        self.runtime = EngineRuntime(engine_config, device)
        self.tokenizer = self.runtime.tokenizer
        self._queues: Dict[str, "queue.Queue"] = {}
        self._lock = threading.Lock()
        conv_json = json.dumps(self.runtime.conv_template.to_json_dict())
        self._ffi = _core.JsonFFIEngine(lambda cfg: self.runtime.make_core_engine(cfg, None),
                                        self.tokenizer.handle, conv_json, model, self._on_chunks)
        if hasattr(self.runtime.models[0], "image_embed"):
            self._ffi.set_image_embedder(self._embed_image)
        self._threads = [threading.Thread(target=self._ffi.run_background_loop, daemon=True),
                         threading.Thread(target=self._ffi.run_background_stream_back_loop, daemon=True)]
        for t in self._threads:
            t.start()
        self._ffi.reload(self.runtime.complete_config_json)
        self.chat = _Chat(self)
        self._terminated = False

    def _embed_image(self, image_bytes: bytes):
        """Encoded image bytes (the native side has already taken them out of the data URL) -> embedding rows
        held by the executor: (handle, number of rows)."""
        import io  # pylint: disable=import-outside-toplevel

        from PIL import Image  # pylint: disable=import-outside-toplevel

        from ..models.vision import preprocess_image  # pylint: disable=import-outside-toplevel

        img = Image.open(io.BytesIO(image_bytes)).convert("RGB")
        pixels, _ = preprocess_image(img, self.runtime.models_info[0].chat_config)
        emb = self.runtime.models[0].image_embed(pixels)
        return self.runtime.executor.hold_embedding(emb), int(emb.shape[0])

    def _on_chunks(self, chunks_json: str) -> None:
        for chunk in json.loads(chunks_json):
            with self._lock:
                q = self._queues.get(chunk["id"])
            if q is not None:
                q.put(chunk)

    def _raw_chat_completion(self, request_json: str, include_usage: bool, request_id: str
                             ) -> Iterator[openai.ChatCompletionStreamResponse]:
        q: "queue.Queue" = queue.Queue()
        with self._lock:
            self._queues[request_id] = q
        try:
            if not self._ffi.chat_completion(request_json, request_id):
                raise ValueError(self._ffi.get_last_error())
            while True:
                chunk = q.get()
                final = chunk.get("usage") is not None
                if not final or include_usage:
                    yield openai.ChatCompletionStreamResponse.model_validate(chunk)
                if final:
                    return
        except GeneratorExit:
            self._ffi.abort(request_id)
            raise
        finally:
            with self._lock:
                self._queues.pop(request_id, None)

    def metrics(self) -> Dict[str, Any]:
        return json.loads(self._ffi.json_metrics())

    def terminate(self) -> None:
        if self._terminated:
            return
        self._terminated = True
        self._ffi.exit_background_loop()
        for t in self._threads:
            t.join(timeout=10)

    def _test_reload(self) -> None:
        self._ffi.reload(self.runtime.complete_config_json)

    def _test_reset(self) -> None:
        self._ffi.reset()

    def _test_unload(self) -> None:
        self._ffi.unload()
