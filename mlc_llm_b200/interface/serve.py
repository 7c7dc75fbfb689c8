"""``mlc_llm_b200 serve``: build the engine(s), mount the routers, run uvicorn (reference:
``python/mlc_llm/interface/serve.py:24-131``)."""

from __future__ import annotations

from typing import Any, List, Literal, Optional, Tuple, Union

import fastapi
import uvicorn
from fastapi.middleware.cors import CORSMiddleware

from ..protocol import error_protocol
from ..serve import engine
from ..serve.config import EngineConfig
from ..serve.entrypoints import (debug_entrypoints, metrics_entrypoints, microserving_entrypoints,
                                 openai_entrypoints)
from ..serve.server import ServerContext


def build_app(server_context: ServerContext, *, enable_debug: bool = False, allow_credentials: bool = False,
              allow_origins: Any = ("*",), allow_methods: Any = ("*",), allow_headers: Any = ("*",)
              ) -> fastapi.FastAPI:
    """The FastAPI application over an already populated server context."""
    app = fastapi.FastAPI()
    app.add_middleware(CORSMiddleware, allow_credentials=allow_credentials, allow_origins=list(allow_origins),
                       allow_methods=list(allow_methods), allow_headers=list(allow_headers))
    app.include_router(openai_entrypoints.app)
    app.include_router(metrics_entrypoints.app)
    app.include_router(microserving_entrypoints.app)
    ServerContext.enable_debug = enable_debug
    if enable_debug:
        app.include_router(debug_entrypoints.app)
    app.exception_handler(error_protocol.BadRequestError)(error_protocol.bad_request_error_handler)
    return app


def serve(  # pylint: disable=too-many-arguments,too-many-locals
    model: str,
    device: str = "auto",
    model_lib: Optional[str] = None,
    mode: Literal["local", "interactive", "server"] = "local",
    enable_debug: bool = False,
    additional_models: Optional[List[Union[str, Tuple[str, str]]]] = None,
    embedding_model: Optional[str] = None,
    embedding_model_lib: Optional[str] = None,
    tensor_parallel_shards: Optional[int] = None,
    pipeline_parallel_stages: Optional[int] = None,
    opt: Optional[str] = None,
    max_num_sequence: Optional[int] = None,
    max_total_sequence_length: Optional[int] = None,
    max_single_sequence_length: Optional[int] = None,
    prefill_chunk_size: Optional[int] = None,
    sliding_window_size: Optional[int] = None,
    attention_sink_size: Optional[int] = None,
    max_history_size: Optional[int] = None,
    gpu_memory_utilization: Optional[float] = None,
    speculative_mode: Literal["disable", "small_draft", "eagle", "medusa"] = "disable",
    spec_draft_length: Optional[int] = None,
    spec_tree_width: Optional[int] = None,
    prefix_cache_mode: Literal["disable", "radix"] = "radix",
    prefix_cache_max_num_recycling_seqs: Optional[int] = None,
    prefill_mode: Literal["hybrid", "chunked"] = "hybrid",
    enable_tracing: bool = False,
    host: str = "127.0.0.1",
    port: int = 8000,
    allow_credentials: bool = False,
    allow_origins: Any = ("*",),
    allow_methods: Any = ("*",),
    allow_headers: Any = ("*",),
    api_key: Optional[str] = None,
) -> None:
    cfg = EngineConfig(
        additional_models=list(additional_models or []), tensor_parallel_shards=tensor_parallel_shards,
        pipeline_parallel_stages=pipeline_parallel_stages, opt=opt, max_num_sequence=max_num_sequence,
        max_total_sequence_length=max_total_sequence_length,
        max_single_sequence_length=max_single_sequence_length, prefill_chunk_size=prefill_chunk_size,
        sliding_window_size=sliding_window_size, attention_sink_size=attention_sink_size,
        max_history_size=max_history_size, gpu_memory_utilization=gpu_memory_utilization,
        speculative_mode=speculative_mode, spec_draft_length=spec_draft_length or 0,
        spec_tree_width=spec_tree_width or 1, prefix_cache_mode=prefix_cache_mode,
        prefix_cache_max_num_recycling_seqs=prefix_cache_max_num_recycling_seqs, prefill_mode=prefill_mode)
    async_engine = engine.AsyncMLCEngine(model=model, device=device, model_lib=model_lib, mode=mode,
                                         engine_config=cfg, enable_tracing=enable_tracing)
    emb_engine = None
    if embedding_model is not None:
        from ..serve.embedding_engine import AsyncEmbeddingEngine  # pylint: disable=import-outside-toplevel

        emb_engine = AsyncEmbeddingEngine(embedding_model, model_lib=embedding_model_lib, device=device)
    with ServerContext() as ctx:
        ctx.add_model(model, async_engine)
        if emb_engine is not None:
            ctx.set_embedding_engine(embedding_model, emb_engine)
        ctx.api_key = api_key
        app = build_app(ctx, enable_debug=enable_debug, allow_credentials=allow_credentials,
                        allow_origins=allow_origins, allow_methods=allow_methods, allow_headers=allow_headers)
        uvicorn.run(app, host=host, port=port, log_level="info")
