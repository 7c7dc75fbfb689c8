"""``mlc_llm_b200 router``: an OpenAI ``/v1/completions`` front end over a :class:`Router` (reference:
``python/mlc_llm/interface/router.py:17-130``)."""

from __future__ import annotations

from http import HTTPStatus
from typing import List, Literal, Optional, Type

import fastapi
import uvicorn
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import StreamingResponse

from ..protocol import error_protocol
from ..protocol import openai_api_protocol as openai
from ..router import Router
from ..serve import engine_base


def build_app(router: Router) -> fastapi.FastAPI:
    app = fastapi.FastAPI()
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])

    @app.post("/v1/completions")
    async def request_completion(request: openai.CompletionRequest):
        request_id = engine_base.create_request_id("cmpl", None)
        try:
            gen = router.handle_completion(request, request_id)
            if request.stream:
                first = await gen.__anext__()

                async def stream():
                    if first is not None:
                        yield f"data: {first.model_dump_json(by_alias=True)}\n\n"
                    async for chunk in gen:
                        if chunk is None:
                            continue  # the engine preempted the request; the client may retry
                        yield f"data: {chunk.model_dump_json(by_alias=True)}\n\n"
                    yield "data: [DONE]\n\n"

                return StreamingResponse(stream(), media_type="text/event-stream")
            texts: List[str] = []
            finish = None
            usage = None
            async for chunk in gen:
                if chunk is None:
                    return error_protocol.create_error_response(HTTPStatus.SERVICE_UNAVAILABLE,
                                                                message="The request was preempted; retry.")
                for choice in chunk.choices:
                    while len(texts) <= choice.index:
                        texts.append("")
                    texts[choice.index] += choice.text
                    finish = choice.finish_reason or finish
                usage = chunk.usage or usage
            return openai.CompletionResponse(
                id=request_id, model=request.model, usage=usage,
                choices=[openai.CompletionResponseChoice(index=i, text=t, finish_reason=finish)
                         for i, t in enumerate(texts)])
        except (ValueError, RuntimeError) as err:
            return error_protocol.create_error_response(HTTPStatus.BAD_REQUEST, message=str(err))

    return app


def serve(model: str, model_lib: Optional[str], router_host: str, router_port: int, endpoint_hosts: List[str],
          endpoint_ports: List[int], endpoint_num_gpus: List[int], enable_prefix_cache: bool,
          router_mode: Literal["disagg", "round-robin"] = "round-robin", pd_balance_factor: float = 0.0,
          router_type: Type[Router] = Router, device: str = "cuda") -> None:
    router = router_type(model=model, model_lib=model_lib, hosts=endpoint_hosts, ports=endpoint_ports,
                         num_gpus=endpoint_num_gpus, enable_prefix_cache=enable_prefix_cache,
                         router_mode=router_mode, pd_balance_factor=pd_balance_factor, device=device)
    try:
        uvicorn.run(build_app(router), host=router_host, port=router_port, log_level="info")
    finally:
        router.terminate()
