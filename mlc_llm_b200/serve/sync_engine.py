"""``SyncMLCEngine``: the native engine driven step by step from the calling thread.

No background threads: ``add_request`` queues work and every ``step()`` runs exactly one scheduling
action, which makes engine behaviour deterministic for tests and lets a benchmark bracket a known
number of steps with CUDA events.  Reference: ``python/mlc_llm/serve/sync_engine.py:88-359``.
"""

from __future__ import annotations

import json
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..tokenizers import TextStreamer
from . import engine_base
from .config import EngineConfig
from .data import RequestStreamOutput
from .engine_base import EngineRuntime


class SyncMLCEngine:
    def __init__(self, model: str, device: Union[str, torch.device] = "auto", *,
                 model_lib: Optional[str] = None, mode: str = "local",
                 engine_config: Optional[EngineConfig] = None, enable_tracing: bool = False,
                 request_stream_callback: Optional[Callable[[List[RequestStreamOutput]], None]] = None,
                 comm=None, runtime: Optional[EngineRuntime] = None):
        if runtime is None:
            engine_config = engine_config or EngineConfig()
            engine_config.model = model
            if model_lib is not None:
                engine_config.model_lib = model_lib
            if engine_config.mode is None:
                engine_config.mode = mode
            from .. import _core  # pylint: disable=import-outside-toplevel

            trace = _core.EventTraceRecorder() if enable_tracing else None
            runtime = EngineRuntime(engine_config, device, comm=comm, trace_recorder=trace)
        self.runtime = runtime
        self.trace_recorder = runtime.trace
        self.tokenizer = runtime.tokenizer
        self._user_callback = request_stream_callback
        self._outputs: List[dict] = []
        self._engine = runtime.make_core_engine(None, self._on_outputs)
        self.engine_config = EngineConfig.from_json(self._engine.config_json())
        self._next_id = 0

    def _on_outputs(self, outs: List[dict]) -> None:
        if self._user_callback is not None:
            items = []
            for o in outs:
                o = o if isinstance(o, dict) else o.asdict()
                has_delta = any(o["group_delta_token_ids"]) or any(r is not None for r in o["group_finish_reason"])
                if o["request_final_usage_json_str"] is not None and has_delta:
                    # callers of the callback API expect the usage record in an item of its own, after the
                    # item with the last tokens
                    items.append(RequestStreamOutput(dict(o, request_final_usage_json_str=None)))
                    items.append(RequestStreamOutput(dict(o, group_delta_token_ids=[], group_delta_logprob_json_strs=[],
                                                          group_finish_reason=[], group_extra_prefix_string=[])))
                else:
                    items.append(RequestStreamOutput(o))
            self._user_callback(items)
        else:
            self._outputs.extend(outs)

    # ------------------------------------------------------------------ low-level API
    def create_request(self, request_id: str, inputs, generation_config):
        """A ``Request`` for ``add_request`` (reference: ``serve/sync_engine.py:293``); ``inputs`` is one
        ``Data`` item or a list of them."""
        from .request import Request  # pylint: disable=import-outside-toplevel

        return Request(request_id, inputs if isinstance(inputs, (list, tuple)) else [inputs], generation_config)

    def _native_inputs(self, inputs: Sequence[Any]) -> List[Any]:
        out = []
        for x in inputs:
            if isinstance(x, tuple):
                out.append(x)
            elif isinstance(x, str) or hasattr(x, "text"):
                out.append(np.asarray(self.tokenizer.encode(x if isinstance(x, str) else x.text), dtype=np.int32))
            elif hasattr(x, "token_ids"):
                out.append(np.asarray(x.token_ids, dtype=np.int32))
            elif hasattr(x, "embed_size"):  # ImageData -> embedding rows held by the executor
                model = self.runtime.models[0]
                if not hasattr(model, "image_embed"):
                    raise ValueError("this model does not take image inputs")
                emb = model.image_embed(x.image)
                out.append(("embed", self.runtime.executor.hold_embedding(emb), int(emb.shape[0])))
            else:
                out.append(np.asarray(x, dtype=np.int32))
        return out

    def add_request(self, request_id, inputs: Optional[Sequence[Any]] = None,
                    generation_config: Optional[Dict[str, Any]] = None) -> None:
        """``add_request(request)`` with a ``Request`` from ``create_request``, or
        ``add_request(request_id, inputs, generation_config)``."""
        if inputs is None and hasattr(request_id, "inputs"):
            request_id, inputs, generation_config = (request_id.request_id, request_id.inputs,
                                                     request_id.generation_config)
        cfg = generation_config or {}
        if not isinstance(cfg, dict):
            cfg = cfg.model_dump(exclude_none=True) if hasattr(cfg, "model_dump") else dict(vars(cfg))
        self._engine.add_request(request_id, self._native_inputs(inputs), json.dumps(cfg))

    def abort_request(self, request_id: str) -> None:
        self._engine.abort_request(request_id)

    def step(self) -> None:
        self._engine.step()

    def empty(self) -> bool:
        return self._engine.empty()

    def reset(self) -> None:
        self._engine.reset()

    def metrics(self) -> Dict[str, Any]:
        return json.loads(self._engine.json_metrics())

    def debug_stats(self) -> str:
        return self._engine.debug_stats()

    def take_outputs(self) -> List[dict]:
        outs, self._outputs = self._outputs, []
        return outs

    # ------------------------------------------------------------------ conveniences
    def generate(self, prompts: Sequence[Union[str, List[int]]], generation_config: Union[Dict[str, Any], List[Dict[str, Any]]]
                 ) -> Tuple[List[List[str]], List[List[List[int]]]]:
        """Run all prompts to completion. Returns (texts[request][choice], token_ids[request][choice])."""
        n_req = len(prompts)
        cfgs = generation_config if isinstance(generation_config, list) else [generation_config] * n_req
        ids = []
        for p, g in zip(prompts, cfgs):
            rid = f"sync-{self._next_id}"
            self._next_id += 1
            ids.append(rid)
            toks = self.tokenizer.encode(p) if isinstance(p, str) else list(p)
            self.add_request(rid, [toks], g)
        index = {rid: i for i, rid in enumerate(ids)}
        tokens: List[List[List[int]]] = [[[] for _ in range(int(g.get("n", 1)))] for g in cfgs]
        streamers = [[TextStreamer(self.tokenizer) for _ in req] for req in tokens]
        texts = [["" for _ in req] for req in tokens]
        while not self.empty():
            self.step()
            for out in self.take_outputs():
                i = index.get(out["request_id"])
                if i is None:
                    continue
                for c, delta in enumerate(out["group_delta_token_ids"]):
                    tokens[i][c].extend(delta)
                    # grammar-forced text (jump-forward decoding) is delivered as a string, not as ids
                    extra = out["group_extra_prefix_string"][c]
                    if extra and out["group_finish_reason"][c] != "error":
                        texts[i][c] += extra
                    if delta:
                        texts[i][c] += streamers[i][c].put(delta)
        for i, req in enumerate(texts):
            for c in range(len(req)):
                req[c] += streamers[i][c].finish()
        return texts, tokens

    def run_token_workload(self, prompts: List[List[int]], generation_config: Dict[str, Any]) -> int:
        """Benchmark driver: submit token-id prompts, step until drained, return the number of output
        tokens produced (counted from the engine's final usage records)."""
        cfg_json = generation_config
        for p in prompts:
            rid = f"wl-{self._next_id}"
            self._next_id += 1
            self.add_request(rid, [p], cfg_json)
        produced = 0
        while not self.empty():
            self.step()
            for out in self._outputs:
                usage = out["request_final_usage_json_str"]
                if usage is not None:
                    produced += json.loads(usage)["completion_tokens"]
            self._outputs.clear()
        return produced
