"""Programmable request router over several server processes (reference:
``python/mlc_llm/router/router.py:21-390``).

Two policies:

* ``round-robin``: every request goes whole to the endpoint with the fewest requests in flight;
* ``disagg``: endpoint 0 prefills, the others decode.  Per request: ``prep_recv`` on a decode endpoint
  (reserve KV, learn the prefix-cache hit), ``remote_send`` on the prefill endpoint (compute the
  missing KV and copy it into the decode engine's pages over NVLink), ``start_generate`` on the
  decode endpoint.  ``pd_balance_factor`` leaves that fraction of the prompt to be prefilled by the
  decode endpoint itself.  A reply that finishes with ``preempt`` is surfaced as ``None`` so the
  caller can retry.

Endpoints are started on disjoint GPU ranges of one box; the peer-copy group description they need
travels in ``MLCB_DISAGG_GROUP`` (the counterpart of the reference's NVSHMEM uid hand-off).
"""

from __future__ import annotations

import json
import math
import threading
from typing import Any, AsyncGenerator, Iterable, List, Literal, Optional, Tuple

import aiohttp

from ..protocol import openai_api_protocol as openai
from ..protocol.microserving_protocol import PrepRecvRequest, RemoteSendRequest, StartGenerateRequest
from ..serve.config import EngineConfig
from ..serve.server import PopenServer


class Router:  # pylint: disable=too-many-instance-attributes
    def __init__(self, model: str, model_lib: Optional[str] = None, hosts: Optional[List[str]] = None,
                 ports: Optional[List[int]] = None, num_gpus: Optional[List[int]] = None,
                 enable_prefix_cache: bool = False, router_mode: Literal["disagg", "round-robin"] = "disagg",
                 pd_balance_factor: float = 0.0, device: str = "cuda", start_servers: bool = True,
                 server_start_timeout: float = 900.0, api_key: Optional[str] = None):
        hosts = hosts or ["127.0.0.1"]
        ports = ports or [8080]
        num_gpus = num_gpus or [1]
        if not len(hosts) == len(ports) == len(num_gpus):
            raise ValueError("hosts, ports and num_gpus must have one entry per endpoint")
        if router_mode == "disagg" and len(hosts) < 2:
            raise ValueError("disaggregated routing needs a prefill endpoint and at least one decode endpoint")
        self.model = model
        self.router_mode = router_mode
        self.pd_balance_factor = pd_balance_factor
        self.num_servers = len(hosts)
        self.server_urls = [f"http://{h}:{p}" for h, p in zip(hosts, ports)]
        self.headers = {"Content-Type": "application/json"}
        if api_key:  # the endpoints' microserving routes sit behind the same key as their OpenAI routes
            self.headers["Authorization"] = f"Bearer {api_key}"
        self.num_running_requests = [0] * self.num_servers
        self.device_id_starts = [0]
        for n in num_gpus:
            self.device_id_starts.append(self.device_id_starts[-1] + n)
        self.servers: List[PopenServer] = []
        if start_servers:
            group = {"world": self.device_id_starts[-1], "starts": self.device_id_starts[:-1]}
            errors: List[BaseException] = []

            def start(i: int) -> None:
                gpu_ids = list(range(self.device_id_starts[i], self.device_id_starts[i + 1])) \
                    if device.startswith("cuda") else None
                server_device = device
                if router_mode == "disagg" and device.startswith("cuda"):
                    # the prefill engine maps the decode engine's KV pool through CUDA IPC, so every
                    # endpoint must see all GPUs: select the device by index instead of masking
                    gpu_ids = None
                    server_device = f"cuda:{self.device_id_starts[i]}"
                srv = PopenServer(
                    model, server_device, model_lib=model_lib, mode="server", host=hosts[i], port=ports[i],
                    enable_debug=True, gpu_ids=gpu_ids, api_key=api_key,
                    tensor_parallel_shards=num_gpus[i] if num_gpus[i] > 1 else None,
                    engine_config=EngineConfig(prefix_cache_mode="radix" if enable_prefix_cache else "disable",
                                               gpu_memory_utilization=0.8),
                    extra_env={"MLCB_DISAGG_GROUP": json.dumps(dict(group, index=i))})
                self.servers.append(srv)
                try:
                    srv.start(timeout=server_start_timeout)
                except BaseException as err:  # pylint: disable=broad-except
                    errors.append(err)

            threads = [threading.Thread(target=start, args=(i,)) for i in range(self.num_servers)]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
            if errors:
                self.terminate()
                raise errors[0]

    def terminate(self) -> None:
        for srv in self.servers:
            srv.terminate()
        self.servers = []

    # ------------------------------------------------------------------ dispatch
    def translate_request(self, request: openai.CompletionRequest, request_id: str):
        """The reference's name for ``handle_completion`` (``router/router.py:134``)."""
        return self.handle_completion(request, request_id)

    async def handle_completion(self, request: openai.CompletionRequest, request_id: str
                                ) -> AsyncGenerator[Optional[openai.CompletionResponse], Any]:
        if isinstance(request.prompt, str):
            raise ValueError("the router expects token-id prompts (tokenise before routing)")
        if self.router_mode == "disagg":
            async for chunk in self._handle_completion_disagg(request, request_id, self.pd_balance_factor):
                yield chunk
        elif self.router_mode == "round-robin":
            async for chunk in self._handle_completion_round_robin(request):
                yield chunk
        else:
            raise ValueError(f"unknown router mode {self.router_mode}")

    def _pick_endpoint(self, endpoint_ids: Iterable[int]) -> int:
        """The endpoint with the fewest requests in flight (first wins ties)."""
        best, best_load = -1, None
        for i in endpoint_ids:
            if best_load is None or self.num_running_requests[i] < best_load:
                best, best_load = i, self.num_running_requests[i]
        if best < 0:
            raise RuntimeError("no endpoint to pick from")
        return best

    @staticmethod
    async def _stream_chunks(response: aiohttp.ClientResponse) -> AsyncGenerator[openai.CompletionResponse, Any]:
        async for line in response.content:
            line = line.strip()
            if not line.startswith(b"data:"):
                continue
            body = line[5:].strip()
            if body == b"[DONE]":
                continue
            yield openai.CompletionResponse.model_validate(json.loads(body))

    @staticmethod
    def _preempted(resp: openai.CompletionResponse) -> bool:
        return bool(resp.choices) and resp.choices[0].finish_reason == "preempt"

    async def _handle_completion_round_robin(self, request: openai.CompletionRequest
                                             ) -> AsyncGenerator[Optional[openai.CompletionResponse], Any]:
        endpoint = self._pick_endpoint(range(self.num_servers))
        self.num_running_requests[endpoint] += 1
        try:
            payload = request.model_dump(by_alias=True)
            timeout = aiohttp.ClientTimeout(total=3 * 3600)
            async with aiohttp.ClientSession(timeout=timeout, trust_env=True) as session:
                async with session.post(self.server_urls[endpoint] + "/v1/completions", json=payload,
                                        headers=self.headers) as response:
                    if response.status != 200:
                        raise RuntimeError(await response.text())
                    if payload.get("stream"):
                        async for chunk in self._stream_chunks(response):
                            if self._preempted(chunk):
                                yield None
                            yield chunk
                    else:
                        chunk = openai.CompletionResponse.model_validate(await response.json())
                        if self._preempted(chunk):
                            yield None
                        yield chunk
        finally:
            self.num_running_requests[endpoint] -= 1

    async def _handle_completion_disagg(self, original: openai.CompletionRequest, request_id: str,
                                        pd_balance_factor: float = 0.0
                                        ) -> AsyncGenerator[Optional[openai.CompletionResponse], Any]:
        original.user = request_id  # the three steps must name the same engine request
        prefill_id = 0
        decode_id = self._pick_endpoint(range(1, self.num_servers))
        prompt_len = len(original.prompt)
        kv_window_end = -1 if math.fabs(pd_balance_factor) < 1e-5 else int((1 - pd_balance_factor) * prompt_len)
        self.num_running_requests[decode_id] += 1
        try:
            timeout = aiohttp.ClientTimeout(total=3 * 3600)
            async with aiohttp.ClientSession(timeout=timeout, trust_env=True) as session:
                base = original.model_dump(by_alias=True)
                metadata, matched = await self.send_prepare_receive(
                    session, PrepRecvRequest(**base, end=kv_window_end), self.server_urls[decode_id])
                if kv_window_end < 0:
                    kv_window_end = prompt_len + kv_window_end
                if matched > kv_window_end:
                    raise RuntimeError("decode endpoint matched more of the prompt than it was asked to receive")
                if matched < kv_window_end:
                    await self.send_remote_send(
                        session,
                        RemoteSendRequest(**base, begin=matched, end=kv_window_end, kv_addr_info=metadata,
                                          recv_rank=self.device_id_starts[decode_id]),
                        self.server_urls[prefill_id])
                async for chunk in self.send_start_generate(
                        session, StartGenerateRequest(**base, begin=kv_window_end), self.server_urls[decode_id]):
                    if self._preempted(chunk):
                        yield None
                    yield chunk
        finally:
            self.num_running_requests[decode_id] -= 1

    async def send_prepare_receive(self, session: aiohttp.ClientSession, request: PrepRecvRequest,
                                   server_url: str) -> Tuple[str, int]:
        async with session.post(server_url + "/microserving/prep_recv", json=request.model_dump(by_alias=True),
                                headers=self.headers) as response:
            if response.status != 200:
                raise RuntimeError(await response.text())
            data = await response.json()
            return data["kv_append_metadata"], int(data["prefix_matched_length"])

    async def send_remote_send(self, session: aiohttp.ClientSession, request: RemoteSendRequest,
                               server_url: str) -> None:
        async with session.post(server_url + "/microserving/remote_send", json=request.model_dump(by_alias=True),
                                headers=self.headers) as response:
            if response.status != 200:
                raise RuntimeError(await response.text())
            await response.json()

    async def send_start_generate(self, session: aiohttp.ClientSession, request: StartGenerateRequest,
                                  server_url: str) -> AsyncGenerator[openai.CompletionResponse, Any]:
        async with session.post(server_url + "/microserving/start_generate",
                                json=request.model_dump(by_alias=True), headers=self.headers) as response:
            if response.status != 200:
                raise RuntimeError(await response.text())
            if request.stream:
                async for chunk in self._stream_chunks(response):
                    yield chunk
            else:
                yield openai.CompletionResponse.model_validate(await response.json())
