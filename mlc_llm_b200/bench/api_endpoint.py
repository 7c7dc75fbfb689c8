"""HTTP clients of the load generator (reference: ``python/mlc_llm/bench/api_endpoint.py``).
Each sends one request, streams the reply, and fills the record's client-side timings: TTFT is the
time to the first non-empty content chunk."""

from __future__ import annotations

import json
import time
from typing import Optional

import aiohttp

from .request_record import Metrics, RequestRecord, ServerMetrics


class APIEndPoint:
    def __init__(self, include_server_metrics: bool = False):
        self.include_server_metrics = include_server_metrics

    async def __aenter__(self):
        return self

    async def __aexit__(self, *exc):
        return None

    async def __call__(self, record: RequestRecord) -> RequestRecord:
        raise NotImplementedError


class OpenAIEndPoint(APIEndPoint):
    """``/v1/chat/completions`` for message prompts, ``/v1/completions`` for token-id prompts."""

    def __init__(self, host: str, port: int, timeout: Optional[float] = None,
                 include_server_metrics: bool = False, api_key: Optional[str] = None, model: str = ""):
        super().__init__(include_server_metrics)
        self.base = f"http://{host}:{port}"
        self.timeout = timeout
        self.model = model
        self.headers = {"Content-Type": "application/json"}
        if api_key:
            self.headers["Authorization"] = f"Bearer {api_key}"
        self.session: Optional[aiohttp.ClientSession] = None

    async def __aenter__(self):
        self.session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout), trust_env=True)
        return self

    async def __aexit__(self, *exc):
        if self.session is not None:
            await self.session.close()
            self.session = None

    async def __call__(self, record: RequestRecord) -> RequestRecord:  # pylint: disable=too-many-branches,too-many-locals
        body = dict(record.chat_cmpl)
        body["model"] = body.get("model") or self.model
        body["stream"] = True
        body["stream_options"] = {"include_usage": True}
        if record.input_token_ids is not None:
            url = self.base + "/v1/completions"
            body.pop("messages", None)
            body["prompt"] = record.input_token_ids
        else:
            url = self.base + "/v1/chat/completions"
        text, first_chunk = "", ""
        ttft = None
        usage = None
        start = time.monotonic()
        try:
            async with self.session.post(url, json=body, headers=self.headers) as resp:
                if resp.status != 200:
                    raise RuntimeError(f"HTTP {resp.status}: {await resp.text()}")
                async for line in resp.content:
                    line = line.strip()
                    if not line.startswith(b"data:"):
                        continue
                    payload = line[5:].strip()
                    if payload == b"[DONE]":
                        break
                    data = json.loads(payload)
                    if data.get("usage"):
                        usage = data["usage"]
                    for choice in data.get("choices", []):
                        piece = choice.get("text")
                        if piece is None:
                            piece = (choice.get("delta") or {}).get("content") or ""
                        if piece and ttft is None:
                            ttft = time.monotonic() - start
                            first_chunk = piece
                        text += piece
            finish = time.monotonic()
        except Exception as err:  # pylint: disable=broad-except
            finish = time.monotonic()
            record.error_msg = str(err)
            record.metrics = Metrics(success=False, start_time=start, finish_time=finish,
                                     end_to_end_latency_s=finish - start)
            return record
        record.output_str = text
        record.first_chunk_output_str = first_chunk
        server = None
        if usage and self.include_server_metrics and usage.get("extra"):
            ex = usage["extra"]
            server = ServerMetrics(
                input_tokens=usage.get("prompt_tokens", 0), prefill_tokens=ex.get("prefill_tokens", 0),
                output_tokens=usage.get("completion_tokens", 0),
                end_to_end_latency_s=ex.get("end_to_end_latency_s", 0.0),
                prefill_tokens_per_s=ex.get("prefill_tokens_per_s", 0.0),
                inter_token_latency_s=ex.get("inter_token_latency_s", 0.0),
                time_per_output_token_s=1.0 / ex["decode_tokens_per_s"] if ex.get("decode_tokens_per_s") else 0.0,
                time_to_first_token_s=ex.get("ttft_s"))
        record.metrics = Metrics(
            success=True, start_time=start, finish_time=finish, end_to_end_latency_s=finish - start,
            input_tokens=usage.get("prompt_tokens") if usage else None,
            output_tokens=usage.get("completion_tokens") if usage else None,
            time_to_first_token_s=ttft, server_metrics=server)
        return record


SUPPORTED_BACKENDS = ["openai", "openai-chat", "mlc"]


def create_api_endpoint(args) -> APIEndPoint:
    if args.api_endpoint in SUPPORTED_BACKENDS:
        return OpenAIEndPoint(args.host, args.port, args.timeout, args.include_server_metrics,
                              model=getattr(args, "model", "") or "")
    raise ValueError(f"unknown api endpoint {args.api_endpoint}")
