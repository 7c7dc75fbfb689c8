"""OpenAI-compatible endpoints: ``/v1/models``, ``/v1/completions``, ``/v1/chat/completions``,
``/v1/embeddings`` (reference: ``python/mlc_llm/serve/entrypoints/openai_entrypoints.py:29-340``).

Streaming responses are server-sent events, one ``data: <json>\\n\\n`` per chunk and a final
``data: [DONE]\\n\\n``; a client that disconnects aborts its request in the engine."""

from __future__ import annotations

import base64
import struct
from http import HTTPStatus
from typing import AsyncGenerator, Optional

import fastapi
from fastapi.responses import StreamingResponse

from ...protocol import error_protocol
from ...protocol import openai_api_protocol as openai
from .. import engine_base
from ..server.server_context import ServerContext


async def _check_api_key(request: fastapi.Request) -> None:
    ctx = ServerContext.current()
    key = ctx.api_key if ctx is not None else None
    if not key:
        return
    auth = request.headers.get("Authorization", "")
    if auth != f"Bearer {key}":
        raise fastapi.HTTPException(status_code=HTTPStatus.UNAUTHORIZED.value, detail="Invalid or missing API key")


app = fastapi.APIRouter(dependencies=[fastapi.Depends(_check_api_key)])


def _no_engine(model: Optional[str]):
    return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST,
                                                message=f'The requested model "{model}" is not served.')


@app.get("/v1/models")
async def list_models() -> openai.ListResponse:
    ctx = ServerContext.current()
    return openai.ListResponse(data=[openai.ModelResponse(id=m) for m in ctx.get_model_list()])


def _debug_enabled() -> bool:
    return bool(ServerContext.enable_debug)


def _strip_debug(request) -> None:
    """Without ``--enable-debug`` a client cannot set debug options (ignore_eos, pinned system prompts,
    special requests, the disaggregation controls): the field is dropped before the engine sees it
    (reference: ``openai_entrypoints.py:139-143,243-247``)."""
    if not _debug_enabled():
        request.debug_config = None


def _public(response):
    """Engine-internal statistics in ``usage.extra`` are for debug servers only."""
    usage = getattr(response, "usage", None)
    if usage is not None and getattr(usage, "extra", None) is not None and not _debug_enabled():
        usage.extra = None
    return response


async def _sse(gen: AsyncGenerator, first) -> AsyncGenerator[str, None]:
    yield f"data: {_public(first).model_dump_json(by_alias=True, exclude_none=False)}\n\n"
    async for chunk in gen:
        yield f"data: {_public(chunk).model_dump_json(by_alias=True, exclude_none=False)}\n\n"
    yield "data: [DONE]\n\n"


async def _serve_stream(gen: AsyncGenerator):
    """Pull the first chunk before answering, so request errors become HTTP errors instead of a
    broken event stream."""
    try:
        first = await gen.__anext__()
    except StopAsyncIteration:
        async def empty():
            yield "data: [DONE]\n\n"
        return StreamingResponse(empty(), media_type="text/event-stream")
    return StreamingResponse(_sse(gen, first), media_type="text/event-stream")


@app.post("/v1/completions")
async def request_completion(request: openai.CompletionRequest, raw_request: fastapi.Request):
    ctx = ServerContext.current()
    engine = ctx.get_engine(request.model)
    if engine is None:
        return _no_engine(request.model)
    request_id = engine_base.create_request_id("cmpl", request.user)
    _strip_debug(request)
    try:
        if request.stream:
            return await _serve_stream(engine._handle_completion(request, request_id))  # pylint: disable=protected-access
        task = engine._gather_completion(request, request_id)  # pylint: disable=protected-access
        return await _await_or_abort(task, raw_request, engine, request_id)
    except error_protocol.BadRequestError as err:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message=str(err))
    except error_protocol.RequestFailedError as err:
        return error_protocol.create_error_response(HTTPStatus.INTERNAL_SERVER_ERROR, message=str(err))


@app.post("/v1/chat/completions")
async def request_chat_completion(request: openai.ChatCompletionRequest, raw_request: fastapi.Request):
    ctx = ServerContext.current()
    engine = ctx.get_engine(request.model)
    if engine is None:
        return _no_engine(request.model)
    request_id = engine_base.create_request_id("chatcmpl", request.user)
    _strip_debug(request)
    try:
        if request.stream:
            return await _serve_stream(engine._handle_chat_completion(request, request_id))  # pylint: disable=protected-access
        task = engine._gather_chat(request, request_id)  # pylint: disable=protected-access
        return await _await_or_abort(task, raw_request, engine, request_id)
    except error_protocol.BadRequestError as err:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message=str(err))


async def _await_or_abort(coro, raw_request: fastapi.Request, engine, request_id: str):
    """Run a non-streaming request while watching for the client going away."""
    import asyncio  # pylint: disable=import-outside-toplevel

    task = asyncio.ensure_future(coro)
    while True:
        done, _ = await asyncio.wait({task}, timeout=0.5)
        if done:
            return _public(task.result())
        if await raw_request.is_disconnected():
            task.cancel()
            await engine.abort(request_id)
            return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message="The client disconnected.")


@app.post("/v1/embeddings")
async def request_embeddings(request: openai.EmbeddingRequest):
    ctx = ServerContext.current()
    engine = ctx.get_embedding_engine(request.model)
    if engine is None:
        return error_protocol.create_error_response(
            HTTPStatus.BAD_REQUEST, message="No embedding model is served (start the server with --embedding-model).")
    inputs = request.input
    if isinstance(inputs, str):
        inputs = [inputs]
    elif inputs and isinstance(inputs[0], int):
        inputs = [inputs]
    vectors, num_tokens = await engine.async_embed(list(inputs))
    if request.dimensions is not None:
        vectors = [engine.truncate(v, request.dimensions) for v in vectors]
    data = []
    for i, vec in enumerate(vectors):
        if request.encoding_format == "base64":
            emb = base64.b64encode(struct.pack(f"<{len(vec)}f", *vec)).decode("ascii")
        else:
            emb = [float(x) for x in vec]
        data.append(openai.EmbeddingObject(embedding=emb, index=i))
    return openai.EmbeddingResponse(data=data, model=request.model or "",
                                    usage=openai.EmbeddingUsage(prompt_tokens=num_tokens, total_tokens=num_tokens))
