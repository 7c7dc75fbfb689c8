"""``/debug/*`` endpoints, mounted only with ``--enable-debug`` (reference:
``python/mlc_llm/serve/entrypoints/debug_entrypoints.py:16-128``)."""

import json
from http import HTTPStatus

import fastapi
import torch

from ...protocol import error_protocol
from ..server.server_context import ServerContext

app = fastapi.APIRouter()


async def _body(request: fastapi.Request):
    raw = (await request.body()).decode("utf-8")
    try:
        return json.loads(raw) if raw else {}, raw
    except json.JSONDecodeError:
        return None, raw


@app.post("/debug/dump_event_trace")
async def dump_event_trace(request: fastapi.Request):
    body, raw = await _body(request)
    if body is None or "model" not in body:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message=f"Invalid request {raw}")
    engine = ServerContext.current().get_engine(body["model"])
    if engine is None:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST,
                                                    message=f'The requested model "{body["model"]}" is not served.')
    if engine.trace_recorder is None:
        return error_protocol.create_error_response(
            HTTPStatus.BAD_REQUEST, message="Tracing is off; start the server with --enable-tracing.")
    return json.loads(engine.trace_recorder.dump_json())


@app.post("/debug/cuda_profiler_start")
async def cuda_profiler_start(_request: fastapi.Request):
    if torch.cuda.is_available():
        torch.cuda.cudart().cudaProfilerStart()
    return {}


@app.post("/debug/cuda_profiler_stop")
async def cuda_profiler_stop(_request: fastapi.Request):
    if torch.cuda.is_available():
        torch.cuda.cudart().cudaProfilerStop()
    return {}


@app.post("/debug/dump_engine_metrics")
async def dump_engine_metrics(request: fastapi.Request):
    body, raw = await _body(request)
    if body is None:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message=f"Invalid request {raw}")
    engine = ServerContext.current().get_engine(body.get("model"))
    if engine is None:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message="The requested model is not served.")
    return (await engine.metrics()).metrics


@app.post("/debug/reset_engine")
async def reset_engine(request: fastapi.Request):
    body, raw = await _body(request)
    if body is None or "model" not in body:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message=f"Invalid request {raw}")
    engine = ServerContext.current().get_engine(body["model"])
    if engine is None:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message="The requested model is not served.")
    engine.reset()
    return {}
