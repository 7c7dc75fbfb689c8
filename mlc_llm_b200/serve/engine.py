"""``MLCEngine`` and ``AsyncMLCEngine``: OpenAI-style Python API over the native threaded engine.

Reference: ``python/mlc_llm/serve/engine.py`` (:819-1389 async engine, :1391-1946 sync engine;
``chat.completions.create`` / ``completions.create`` with stream and non-stream forms, ``abort``,
``metrics``, ``terminate``, ``reset``).
"""

from __future__ import annotations

import asyncio
import json
import os
import queue
import sys
import threading
from typing import Any, AsyncGenerator, Dict, Iterator, List, Literal, Optional, Union

import torch

from .. import _core
from ..protocol import openai_api_protocol as openai
from ..protocol.error_protocol import BadRequestError
from ..tokenizers import TextStreamer
from . import engine_base
from .config import EngineConfig
from .engine_base import EngineRuntime


class EngineMetrics:
    """Parsed engine metrics with a Prometheus text view."""

    def __init__(self, metrics: Dict[str, Any]):
        self.metrics = metrics

    def __getitem__(self, key):
        return self.metrics[key]

    def prometheus_text(self) -> str:
        return engine_base.metrics_to_prometheus_text(self.metrics)


class _StreamItem:
    """What one callback delivers for one choice of one request."""

    __slots__ = ("delta_text", "delta_logprob_json_strs", "finish_reason", "usage_json", "index")

    def __init__(self, index, delta_text, logprobs, finish_reason, usage_json):
        self.index = index
        self.delta_text = delta_text
        self.delta_logprob_json_strs = logprobs
        self.finish_reason = finish_reason
        self.usage_json = usage_json


class _RequestSink:
    """Per-request state on the frontend: text streamers and the delivery queue."""

    def __init__(self, n: int, tokenizer, deliver):
        self.streamers = [TextStreamer(tokenizer) for _ in range(n)]
        self.deliver = deliver
        self.done = [False] * n


class MLCEngineBase:
    """Owns the runtime (weights, KV cache, executor), the native threaded engine and its two
    background threads."""

    def __init__(self, kind: str, model: str, device: Union[str, torch.device] = "auto", *,
                 model_lib: Optional[str] = None, mode: Literal["local", "interactive", "server"] = "local",
                 engine_config: Optional[EngineConfig] = None, enable_tracing: bool = False, comm=None,
                 runtime: Optional[EngineRuntime] = None):
        self.kind = kind
        self._workers = None
        if runtime is not None:
            self.runtime = runtime
            self.trace_recorder = runtime.trace
        else:
            if engine_config is None:
                engine_config = EngineConfig()
            if engine_config.model is not None and engine_config.model != model:
                raise ValueError("engine_config.model conflicts with the model argument")
            engine_config.model = model
            if model_lib is not None:
                engine_config.model_lib = model_lib
            if engine_config.mode is None:
                engine_config.mode = mode
            self.trace_recorder = _core.EventTraceRecorder() if enable_tracing else None
            tp = int(engine_config.tensor_parallel_shards or 1)
            pp = int(engine_config.pipeline_parallel_stages or 1)
            if comm is None and tp * pp > 1:
                from ..parallel import launcher  # pylint: disable=import-outside-toplevel

                self._workers = launcher.launch(engine_config, engine_base.detect_device(device), tp, pp)
                comm = self._workers.comm
                device = comm.device
            self.runtime = EngineRuntime(engine_config, device, comm=comm, trace_recorder=self.trace_recorder)
        self.tokenizer = self.runtime.tokenizer
        self.conv_template = self.runtime.conv_template
        self.model = model
        self._sinks: Dict[str, _RequestSink] = {}
        self._sinks_lock = threading.Lock()
        self._terminated = False
        self._threaded = _core.ThreadedEngine(self._factory, self._on_outputs)
        self._threads = [
            threading.Thread(target=self._threaded.run_background_loop, daemon=True, name="mlc-engine-loop"),
            threading.Thread(target=self._threaded.run_background_stream_back_loop, daemon=True,
                             name="mlc-stream-back"),
        ]
        # The engine loop and the stream-back loop both run Python (kernel launches, per-request delivery).
        # With CPython's default 5 ms switch interval a burst of deliveries can hold the interpreter lock
        # for its whole length while the engine loop waits to launch the next step; a shorter interval
        # bounds that wait (MLCB_SWITCH_INTERVAL_S, default 0.0005; 0 leaves the interpreter's setting).
        interval = float(os.environ.get("MLCB_SWITCH_INTERVAL_S", "0.0005"))
        if interval > 0 and sys.getswitchinterval() > interval:
            sys.setswitchinterval(interval)
        for t in self._threads:
            t.start()
        self._threaded.reload(self.runtime.complete_config_json)
        self.engine_config = EngineConfig.from_json(self._threaded.get_complete_engine_config())
        self.max_input_sequence_length = int(self.engine_config.max_single_sequence_length or (1 << 30))

    # ---------------------------------------------------------------- native glue
    def _factory(self, engine_config_json: str):
        self._core_engine = self.runtime.make_core_engine(engine_config_json, None)
        return self._core_engine

    def debug_step_count(self) -> int:
        """Scheduling steps taken so far (prefill + decode + verify)."""
        st = json.loads(self._core_engine.debug_stats())
        return int(st.get("num_prefill_steps", 0) + st.get("num_decode_steps", 0) + st.get("num_verify_steps", 0))

    @classmethod
    def from_runtime(cls, runtime: EngineRuntime):
        """Build an engine over an already loaded runtime (weights and KV cache are shared, so the
        engines must not generate at the same time)."""
        return cls(runtime.engine_config.model, runtime.device, runtime=runtime)

    def _on_outputs(self, outputs: List[dict]) -> None:
        """Runs on the stream-back thread: detokenise and hand each request its items."""
        for out in outputs:
            rid = out["request_id"]
            if rid == "":
                # engine-wide failure: fail every open request
                with self._sinks_lock:
                    sinks = list(self._sinks.items())
                why = "".join(out["group_extra_prefix_string"][:1])
                for _, sink in sinks:
                    sink.deliver([_StreamItem(i, why, [], "error", None) for i in range(len(sink.streamers))])
                continue
            with self._sinks_lock:
                sink = self._sinks.get(rid)
            if sink is None:
                continue
            items = []
            usage = out["request_final_usage_json_str"]
            final_text = out["text_is_final"]
            for i, (ids, lps, fr, extra) in enumerate(zip(out["group_delta_token_ids"],
                                                           out["group_delta_logprob_json_strs"],
                                                           out["group_finish_reason"],
                                                           out["group_extra_prefix_string"])):
                if sink.done[i]:
                    continue
                if final_text:
                    # merged result of a request accumulated in the native stream-back thread: `extra` is
                    # the complete, already detokenised text of the choice
                    sink.done[i] = True
                    items.append(_StreamItem(i, extra, lps, fr, None))
                    continue
                text = sink.streamers[i].put(ids) if ids else ""
                if extra and fr != "error":
                    # grammar-forced text (jump-forward decoding) arrives as a string, before the ids
                    text = extra + text
                if fr is not None:
                    text += sink.streamers[i].finish()
                    sink.done[i] = True
                    if fr == "error" and extra:
                        text = extra
                if text or fr is not None or lps:
                    items.append(_StreamItem(i, text, lps, fr, None))
            if usage is not None:
                items.append(_StreamItem(-1, "", [], None, usage))
            if items:
                sink.deliver(items)

    def _register(self, request_id: str, n: int, deliver) -> None:
        with self._sinks_lock:
            if request_id in self._sinks:
                raise BadRequestError(f"The request id {request_id} already exists.")
            self._sinks[request_id] = _RequestSink(n, self.tokenizer, deliver)

    def _unregister(self, request_id: str) -> None:
        with self._sinks_lock:
            self._sinks.pop(request_id, None)

    def _submit(self, request_id: str, inputs: List[Any], gen_cfg: Dict[str, Any]) -> None:
        native_inputs = []
        for item in inputs:
            if hasattr(item, "embed_size"):  # ImageData -> embedding rows held by the executor
                emb = self.runtime.models[0].image_embed(item.image) if hasattr(self.runtime.models[0], "image_embed") \
                    else None
                if emb is None:
                    raise BadRequestError("this model does not take image inputs")
                handle = self.runtime.executor.hold_embedding(emb)
                native_inputs.append(("embed", handle, int(emb.shape[0])))
            else:
                native_inputs.append(item)
        try:
            self._threaded.add_request(request_id, native_inputs, json.dumps(gen_cfg))
        except (ValueError, RuntimeError) as err:
            raise BadRequestError(str(err)) from err

    # ---------------------------------------------------------------- public management API
    def terminate(self) -> None:
        if self._terminated:
            return
        self._terminated = True
        self._threaded.exit_background_loop()
        for t in self._threads:
            t.join(timeout=10)
        workers = getattr(self, "_workers", None)
        if workers is not None:
            workers.shutdown()

    def __del__(self):
        try:
            self.terminate()
        except Exception:  # pylint: disable=broad-except
            pass

    def reset(self) -> None:
        self._threaded.reset()

    def _abort(self, request_id: str) -> None:
        self._threaded.abort_request(request_id)
        self._unregister(request_id)

    def _metrics_json(self) -> Dict[str, Any]:
        return json.loads(self._threaded.json_metrics())


# ====================================================================== async engine
class AsyncChatCompletion:
    def __init__(self, engine: "AsyncMLCEngine"):
        self._engine = engine

    async def create(self, *, messages: List[Dict[str, Any]], model: Optional[str] = None,
                     stream: bool = False, request_id: Optional[str] = None, **kwargs):
        return await self._engine._chat_completion(messages=messages, model=model, stream=stream,
                                                   request_id=request_id, **kwargs)


class AsyncCompletion:
    def __init__(self, engine: "AsyncMLCEngine"):
        self._engine = engine

    async def create(self, *, prompt: Union[str, List[int]], model: Optional[str] = None,
                     stream: bool = False, request_id: Optional[str] = None, **kwargs):
        return await self._engine._completion(prompt=prompt, model=model, stream=stream,
                                              request_id=request_id, **kwargs)


class _Namespace:
    pass


class Chat(_Namespace):
    """``engine.chat``: holds ``completions`` (reference: ``serve/engine.py`` ``Chat``)."""

    def __init__(self, completions=None):
        self.completions = completions


class AsyncChat(Chat):
    """``async_engine.chat`` (reference: ``serve/engine.py`` ``AsyncChat``)."""


class AsyncMLCEngine(MLCEngineBase):
    """Asynchronous engine: many concurrent requests from one asyncio loop."""

    def __init__(self, model: str, device: Union[str, torch.device] = "auto", *,
                 model_lib: Optional[str] = None, mode: Literal["local", "interactive", "server"] = "local",
                 engine_config: Optional[EngineConfig] = None, enable_tracing: bool = False, comm=None,
                 runtime: Optional[EngineRuntime] = None):
        super().__init__("async", model, device, model_lib=model_lib, mode=mode, engine_config=engine_config,
                         enable_tracing=enable_tracing, comm=comm, runtime=runtime)
        self.chat = AsyncChat(AsyncChatCompletion(self))
        self.completions = AsyncCompletion(self)

    async def abort(self, request_id: str) -> None:
        self._abort(request_id)

    async def metrics(self) -> EngineMetrics:
        return EngineMetrics(self._metrics_json())

    # ---------------------------------------------------------------- generation core
    async def _generate(self, inputs: List[Any], gen_cfg: Dict[str, Any], request_id: str,
                        accumulate: bool = False) -> AsyncGenerator[List[_StreamItem], None]:
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()

        def deliver(items):
            loop.call_soon_threadsafe(q.put_nowait, items)

        n = int(gen_cfg.get("n", 1))
        self._register(request_id, n, deliver)
        try:
            if accumulate:  # non-streaming caller: one merged delivery at the end
                self._threaded.accumulate_outputs(request_id, n, self.tokenizer.handle)
            self._submit(request_id, inputs, gen_cfg)
            finished = False
            while not finished:
                items = await q.get()
                finished = any(it.usage_json is not None for it in items) or \
                    any(it.finish_reason == "error" for it in items)
                yield items
        except (asyncio.CancelledError, GeneratorExit):
            self._threaded.abort_request(request_id)
            raise
        finally:
            self._unregister(request_id)

    async def _chat_completion(self, *, messages, model=None, stream=False, request_id=None, **kwargs):
        request = openai.ChatCompletionRequest(messages=messages, model=model, stream=stream, **kwargs)
        rid = request_id or engine_base.create_request_id("chatcmpl", request.user)
        if stream:
            return self._handle_chat_completion(request, rid)
        return await self._gather_chat(request, rid)

    async def _completion(self, *, prompt, model=None, stream=False, request_id=None, **kwargs):
        request = openai.CompletionRequest(prompt=prompt, model=model, stream=stream, **kwargs)
        rid = request_id or engine_base.create_request_id("cmpl", request.user)
        if stream:
            return self._handle_completion(request, rid)
        return await self._gather_completion(request, rid)

    async def _handle_chat_completion(self, request: openai.ChatCompletionRequest, request_id: str
                                      ) -> AsyncGenerator[openai.ChatCompletionStreamResponse, None]:
        inputs, gen, use_fn, _ = engine_base.process_chat_completion_request(
            request, request_id, self.runtime, self.max_input_sequence_length)
        include_usage = request.stream_options is not None and request.stream_options.include_usage
        async for items in self._generate(inputs, gen, request_id):
            chunk = _chat_stream_chunk(items, request_id, self.model, use_fn, include_usage)
            for c in chunk:
                yield c

    async def _handle_completion(self, request: openai.CompletionRequest, request_id: str
                                 ) -> AsyncGenerator[openai.CompletionResponse, None]:
        inputs, gen, _, echo = engine_base.process_completion_request(
            request, request_id, self.runtime, self.max_input_sequence_length)
        include_usage = request.stream_options is not None and request.stream_options.include_usage
        if echo is not None:
            yield openai.CompletionResponse(id=request_id, model=self.model, choices=[
                openai.CompletionResponseChoice(index=i, text=echo) for i in range(request.n)])
        async for items in self._generate(inputs, gen, request_id):
            for c in _completion_stream_chunk(items, request_id, self.model, include_usage, request.legacy_logprobs):
                yield c

    async def _gather_chat(self, request, request_id) -> openai.ChatCompletionResponse:
        inputs, gen, use_fn, _ = engine_base.process_chat_completion_request(
            request, request_id, self.runtime, self.max_input_sequence_length)
        acc = _Accumulator(request.n)
        async for items in self._generate(inputs, gen, request_id, accumulate=True):
            acc.add(items)
        return acc.chat_response(request_id, self.model, use_fn)

    async def _gather_completion(self, request, request_id) -> openai.CompletionResponse:
        inputs, gen, _, echo = engine_base.process_completion_request(
            request, request_id, self.runtime, self.max_input_sequence_length)
        acc = _Accumulator(request.n, echo)
        async for items in self._generate(inputs, gen, request_id, accumulate=True):
            acc.add(items)
        return acc.completion_response(request_id, self.model, request.legacy_logprobs)


# ====================================================================== sync engine
class ChatCompletion:
    def __init__(self, engine: "MLCEngine"):
        self._engine = engine

    def create(self, *, messages: List[Dict[str, Any]], model: Optional[str] = None, stream: bool = False,
               request_id: Optional[str] = None, **kwargs):
        return self._engine._chat_completion(messages=messages, model=model, stream=stream,
                                             request_id=request_id, **kwargs)


class Completion:
    def __init__(self, engine: "MLCEngine"):
        self._engine = engine

    def create(self, *, prompt: Union[str, List[int]], model: Optional[str] = None, stream: bool = False,
               request_id: Optional[str] = None, **kwargs):
        return self._engine._completion(prompt=prompt, model=model, stream=stream, request_id=request_id,
                                        **kwargs)


class MLCEngine(MLCEngineBase):
    """Synchronous engine: one request at a time per calling thread (several threads may call)."""

    def __init__(self, model: str, device: Union[str, torch.device] = "auto", *,
                 model_lib: Optional[str] = None, mode: Literal["local", "interactive", "server"] = "local",
                 engine_config: Optional[EngineConfig] = None, enable_tracing: bool = False, comm=None,
                 runtime: Optional[EngineRuntime] = None):
        super().__init__("sync", model, device, model_lib=model_lib, mode=mode, engine_config=engine_config,
                         enable_tracing=enable_tracing, comm=comm, runtime=runtime)
        self.chat = Chat(ChatCompletion(self))
        self.completions = Completion(self)

    def abort(self, request_id: str) -> None:
        self._abort(request_id)

    def metrics(self) -> EngineMetrics:
        return EngineMetrics(self._metrics_json())

    def _generate(self, inputs: List[Any], gen_cfg: Dict[str, Any], request_id: str,
                  accumulate: bool = False) -> Iterator[List[_StreamItem]]:
        q: "queue.Queue[List[_StreamItem]]" = queue.Queue()
        n = int(gen_cfg.get("n", 1))
        self._register(request_id, n, q.put)
        try:
            if accumulate:  # non-streaming caller: one merged delivery at the end
                self._threaded.accumulate_outputs(request_id, n, self.tokenizer.handle)
            self._submit(request_id, inputs, gen_cfg)
            finished = False
            while not finished:
                items = q.get()
                finished = any(it.usage_json is not None for it in items) or \
                    any(it.finish_reason == "error" for it in items)
                yield items
        except GeneratorExit:
            self._threaded.abort_request(request_id)
            raise
        finally:
            self._unregister(request_id)

    def generate_many(self, prompts: List[List[int]], gen_cfg: Dict[str, Any]) -> List[Dict[str, Any]]:
        """Batch helper: submit token-id prompts together, wait for all, return per-request
        ``{"text", "finish_reason", "usage"}``. Used by offline evaluation and the benchmark."""
        # Results are filled in by the stream-back thread itself; this thread only sleeps until the last
        # request has reported its usage, so it does not compete with the engine loop for the interpreter.
        results = [{"text": "", "finish_reason": None, "usage": None} for _ in prompts]
        done = threading.Event()
        state = {"remaining": len(prompts)}

        def collect(items, i):
            res = results[i]
            for it in items:
                if it.usage_json is not None:
                    res["usage"] = json.loads(it.usage_json)
                    state["remaining"] -= 1
                else:
                    res["text"] += it.delta_text
                    if it.finish_reason is not None:
                        res["finish_reason"] = it.finish_reason
                        if it.finish_reason == "error":
                            state["remaining"] -= 1
            if state["remaining"] <= 0:
                done.set()

        ids = []
        for i, p in enumerate(prompts):
            rid = engine_base.create_request_id("batch", None)
            ids.append(rid)
            self._register(rid, 1, lambda items, i=i: collect(items, i))
        try:
            import numpy as np  # pylint: disable=import-outside-toplevel

            for rid, p in zip(ids, prompts):
                # nobody streams these: let the native stream-back thread gather each request's outputs
                self._threaded.accumulate_outputs(rid, 1, self.tokenizer.handle)
                self._submit(rid, [np.asarray(p, dtype=np.int32)], gen_cfg)
            if prompts:
                done.wait()
        finally:
            for rid in ids:
                self._unregister(rid)
        return results

    def _chat_completion(self, *, messages, model=None, stream=False, request_id=None, **kwargs):
        request = openai.ChatCompletionRequest(messages=messages, model=model, stream=stream, **kwargs)
        rid = request_id or engine_base.create_request_id("chatcmpl", request.user)
        if stream:
            return self._handle_chat_completion(request, rid)
        inputs, gen, use_fn, _ = engine_base.process_chat_completion_request(
            request, rid, self.runtime, self.max_input_sequence_length)
        acc = _Accumulator(request.n)
        for items in self._generate(inputs, gen, rid, accumulate=True):
            acc.add(items)
        return acc.chat_response(rid, self.model, use_fn)

    def _completion(self, *, prompt, model=None, stream=False, request_id=None, **kwargs):
        request = openai.CompletionRequest(prompt=prompt, model=model, stream=stream, **kwargs)
        rid = request_id or engine_base.create_request_id("cmpl", request.user)
        if stream:
            return self._handle_completion(request, rid)
        inputs, gen, _, echo = engine_base.process_completion_request(
            request, rid, self.runtime, self.max_input_sequence_length)
        acc = _Accumulator(request.n, echo)
        for items in self._generate(inputs, gen, rid, accumulate=True):
            acc.add(items)
        return acc.completion_response(rid, self.model, request.legacy_logprobs)

    def _handle_chat_completion(self, request, request_id) -> Iterator[openai.ChatCompletionStreamResponse]:
        inputs, gen, use_fn, _ = engine_base.process_chat_completion_request(
            request, request_id, self.runtime, self.max_input_sequence_length)
        include_usage = request.stream_options is not None and request.stream_options.include_usage
        for items in self._generate(inputs, gen, request_id):
            yield from _chat_stream_chunk(items, request_id, self.model, use_fn, include_usage)

    def _handle_completion(self, request, request_id) -> Iterator[openai.CompletionResponse]:
        inputs, gen, _, echo = engine_base.process_completion_request(
            request, request_id, self.runtime, self.max_input_sequence_length)
        include_usage = request.stream_options is not None and request.stream_options.include_usage
        if echo is not None:
            yield openai.CompletionResponse(id=request_id, model=self.model, choices=[
                openai.CompletionResponseChoice(index=i, text=echo) for i in range(request.n)])
        for items in self._generate(inputs, gen, request_id):
            yield from _completion_stream_chunk(items, request_id, self.model, include_usage, request.legacy_logprobs)


# ====================================================================== response assembly
def _chat_stream_chunk(items, request_id, model, use_fn, include_usage):
    choices, out = [], []
    usage_json = None
    for it in items:
        if it.usage_json is not None:
            usage_json = it.usage_json
            continue
        fr = it.finish_reason
        if use_fn and fr == "stop":
            fr = "tool_calls"
        choices.append(openai.ChatCompletionStreamResponseChoice(
            index=it.index, finish_reason=fr,
            delta=openai.ChatCompletionMessage(content=it.delta_text, role="assistant"),
            logprobs=engine_base.parse_logprobs(it.delta_logprob_json_strs)))
    if choices:
        out.append(openai.ChatCompletionStreamResponse(id=request_id, choices=choices, model=model))
    if usage_json is not None and include_usage:
        out.append(openai.ChatCompletionStreamResponse(id=request_id, choices=[], model=model,
                                                       usage=engine_base.parse_usage(usage_json)))
    return out


def _completion_stream_chunk(items, request_id, model, include_usage, legacy_logprobs=False):
    parse = engine_base.parse_completion_logprobs if legacy_logprobs else engine_base.parse_logprobs
    choices, out = [], []
    usage_json = None
    for it in items:
        if it.usage_json is not None:
            usage_json = it.usage_json
            continue
        fr = it.finish_reason if it.finish_reason in (None, "stop", "length", "preempt") else "stop"
        choices.append(openai.CompletionResponseChoice(index=it.index, finish_reason=fr, text=it.delta_text,
                                                       logprobs=parse(it.delta_logprob_json_strs)))
    if choices:
        out.append(openai.CompletionResponse(id=request_id, choices=choices, model=model))
    if usage_json is not None and include_usage:
        out.append(openai.CompletionResponse(id=request_id, choices=[], model=model,
                                             usage=engine_base.parse_usage(usage_json)))
    return out


class _Accumulator:
    """Collects stream items of a non-streaming request without building per-token objects."""

    def __init__(self, n: int, echo: Optional[str] = None):
        self.texts = [[] if echo is None else [echo] for _ in range(n)]
        self.finish: List[Optional[str]] = [None] * n
        self.logprobs: List[List[str]] = [[] for _ in range(n)]
        self.usage_json: Optional[str] = None

    def add(self, items) -> None:
        for it in items:
            if it.usage_json is not None:
                self.usage_json = it.usage_json
                continue
            if it.delta_text:
                self.texts[it.index].append(it.delta_text)
            if it.delta_logprob_json_strs:
                self.logprobs[it.index].extend(it.delta_logprob_json_strs)
            if it.finish_reason is not None:
                self.finish[it.index] = it.finish_reason

    def chat_response(self, request_id, model, use_fn) -> openai.ChatCompletionResponse:
        texts = ["".join(t) for t in self.texts]
        finish = list(self.finish)
        tool_calls = [None] * len(texts)
        if use_fn:
            ok, calls = engine_base.process_function_call_output(texts, finish)
            if ok:
                tool_calls = calls
        choices = []
        for i, text in enumerate(texts):
            msg = openai.ChatCompletionMessage(role="assistant", content=text) if not tool_calls[i] else \
                openai.ChatCompletionMessage(role="assistant", content=None, tool_calls=tool_calls[i])
            choices.append(openai.ChatCompletionResponseChoice(
                index=i, finish_reason=finish[i], message=msg,
                logprobs=engine_base.parse_logprobs(self.logprobs[i])))
        return openai.ChatCompletionResponse(id=request_id, choices=choices, model=model,
                                             usage=engine_base.parse_usage(self.usage_json))

    def completion_response(self, request_id, model, legacy_logprobs=False) -> openai.CompletionResponse:
        parse = engine_base.parse_completion_logprobs if legacy_logprobs else engine_base.parse_logprobs
        choices = []
        for i, t in enumerate(self.texts):
            if self.finish[i] == "error":
                # the completions protocol has no finish reason for a failed request: the error text the
                # engine put in the stream becomes an exception instead of an empty "stop"
                from ..protocol.error_protocol import RequestFailedError  # pylint: disable=import-outside-toplevel

                raise RequestFailedError("request failed: " + "".join(t))
            fr = self.finish[i] if self.finish[i] in (None, "stop", "length", "preempt") else "stop"
            choices.append(openai.CompletionResponseChoice(
                index=i, finish_reason=fr, text="".join(t),
                logprobs=parse(self.logprobs[i])))
        return openai.CompletionResponse(id=request_id, choices=choices, model=model,
                                         usage=engine_base.parse_usage(self.usage_json))
