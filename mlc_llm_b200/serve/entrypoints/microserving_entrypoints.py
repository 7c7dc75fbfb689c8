"""Prefill/decode disaggregation endpoints (reference:
``python/mlc_llm/serve/entrypoints/microserving_entrypoints.py:22-73``).

Each call is an ordinary completion request whose ``debug_config.disagg_config`` tells the engine
which half of a split request to run:

* ``prep_recv``   - decode engine: match the prompt against its prefix cache, reserve KV pages for
  ``[matched, end)`` and return where a sender may write them;
* ``remote_send`` - prefill engine: compute KV for ``[begin, end)`` and copy the pages into the
  receiver's pool over NVLink peer memory;
* ``start_generate`` - decode engine: prefill ``[begin, len)`` locally and stream the generation.
"""

import json
from http import HTTPStatus

import fastapi

from ...protocol import error_protocol
from ...protocol.debug_protocol import DebugConfig, DisaggConfig
from ...protocol.microserving_protocol import (PrepRecvRequest, PrepRecvResponse, RemoteSendRequest,
                                               RemoteSendResponse, StartGenerateRequest)
from ...protocol.openai_api_protocol import CompletionRequest
from .. import engine_base
from ..server.server_context import ServerContext
from .openai_entrypoints import _check_api_key, _serve_stream

app = fastapi.APIRouter(dependencies=[fastapi.Depends(_check_api_key)])


def _as_completion(request, disagg: DisaggConfig) -> CompletionRequest:
    fields = {k: v for k, v in request.model_dump().items() if k in CompletionRequest.model_fields}
    base = CompletionRequest(**fields)
    if base.debug_config is None:
        base.debug_config = DebugConfig()
    base.debug_config.disagg_config = disagg
    return base


def prep_recv_response(engine, response) -> PrepRecvResponse:
    """Wrap the engine's slot reservation with a handle of its KV pool, so the prefill engine knows
    where (which device memory) and at which slots to write."""
    from .. import kv_handoff  # pylint: disable=import-outside-toplevel

    extra = json.loads(response.usage.extra["disagg"]) if response.usage and response.usage.extra and \
        "disagg" in response.usage.extra else {}
    reservation = json.loads(extra.get("kv_append_metadata") or "{}")
    payload = kv_handoff.encode_payload(engine.runtime.executor.kv_export(0), reservation.get("slots", []),
                                        reservation.get("begin", 0), reservation.get("end", 0))
    return PrepRecvResponse(kv_append_metadata=payload,
                            prefix_matched_length=int(extra.get("prefix_matched_length", 0)))


@app.post("/microserving/prep_recv")
async def prep_recv(request: PrepRecvRequest):
    engine = ServerContext.current().get_engine(request.model)
    if engine is None:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message="The requested model is not served.")
    completion = _as_completion(request, DisaggConfig(kind="prepare_receive", kv_window_begin=0,
                                                      kv_window_end=request.end))
    completion.stream = False
    request_id = engine_base.create_request_id("cmpl", request.user)
    response = await engine._gather_completion(completion, request_id)  # pylint: disable=protected-access
    return prep_recv_response(engine, response)


@app.post("/microserving/remote_send")
async def remote_send(request: RemoteSendRequest):
    engine = ServerContext.current().get_engine(request.model)
    if engine is None:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message="The requested model is not served.")
    completion = _as_completion(request, DisaggConfig(
        kind="remote_send", kv_window_begin=request.begin, kv_window_end=request.end,
        kv_append_metadata=request.kv_addr_info, dst_group_offset=request.recv_rank))
    completion.stream = False
    request_id = engine_base.create_request_id("cmpl", request.user)
    await engine._gather_completion(completion, request_id)  # pylint: disable=protected-access
    return RemoteSendResponse()


@app.post("/microserving/start_generate")
async def start_generate(request: StartGenerateRequest):
    engine = ServerContext.current().get_engine(request.model)
    if engine is None:
        return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message="The requested model is not served.")
    completion = _as_completion(request, DisaggConfig(kind="start_generation", kv_window_begin=request.begin))
    request_id = engine_base.create_request_id("cmpl", request.user)
    if completion.stream:
        return await _serve_stream(engine._handle_completion(completion, request_id))  # pylint: disable=protected-access
    return await engine._gather_completion(completion, request_id)  # pylint: disable=protected-access
