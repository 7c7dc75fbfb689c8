"""Activation calibration: run sampled conversations through the engine and record, per linear layer,
the largest activation magnitude seen at its input (reference: ``python/mlc_llm/interface/calibrate.py``,
whose observer keeps a running ``max`` per parameter name and stores the result in the tensor cache).

The statistics are written as ``<layer>.q_calibration_scale`` (one fp32 value: ``absmax / 448``, the
scale that maps the observed range onto fp8 e4m3) into the tensor cache under ``output``; an existing
cache there is updated in place, so pointing ``output`` at the model directory attaches the scales to
the weights the way the reference does.
"""

from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..loader.tensor_cache import update_tensor_cache

FP8_E4M3_MAX = 448.0


class CalibrationObserver:
    """Running maximum of ``|x|`` per linear layer, keyed by the layer's parameter name."""

    def __init__(self, mode: str = "max"):
        if mode != "max":
            raise NotImplementedError(f"Unsupported calibration mode: {mode}")
        self.names: Dict[int, str] = {}
        self.params: Dict[str, torch.Tensor] = {}

    def watch(self, model) -> None:
        for name, lw in model.p.linears.items():
            self.names[id(lw)] = name

    def __call__(self, lw, x: torch.Tensor) -> None:
        name = self.names.get(id(lw))
        if name is None:
            return
        cur = x.detach().abs().amax().float().reshape(1).cpu()
        prev = self.params.get(name)
        self.params[name] = cur if prev is None else torch.maximum(prev, cur)

    def scales(self) -> List[Tuple[str, torch.Tensor]]:
        return [(f"{n}.q_calibration_scale", (v / FP8_E4M3_MAX).clamp_min(1e-12))
                for n, v in sorted(self.params.items())]

    def save_params(self, output: str) -> None:
        os.makedirs(output, exist_ok=True)
        update_tensor_cache(iter(self.scales()), output, encode_format="raw")


def sample_requests(dataset_path: str, num_requests: int, tokenizer) -> List[Tuple[str, int, int]]:
    """``(prompt, prompt_len, output_len)`` of ``num_requests`` random ShareGPT-style conversations
    (first two turns; 4 <= lengths, prompt <= 1024, total <= 2048 tokens)."""
    with open(dataset_path, encoding="utf-8") as f:
        dataset = json.load(f)
    pairs = [(d["conversations"][0]["value"], d["conversations"][1]["value"])
             for d in dataset if len(d.get("conversations", [])) >= 2]
    kept: List[Tuple[str, int, int]] = []
    for prompt, completion in pairs:
        plen, olen = len(tokenizer.encode(prompt)), len(tokenizer.encode(completion))
        if plen < 4 or olen < 4 or plen > 1024 or plen + olen > 2048:
            continue
        kept.append((prompt, plen, olen))
    if len(kept) < num_requests:
        raise ValueError(f"the dataset has only {len(kept)} usable conversations, {num_requests} requested")
    return random.sample(kept, num_requests)


def calibrate(model: str, device: str, model_lib: Optional[str], dataset: str, output: str,  # pylint: disable=too-many-arguments
              num_calibration_samples: int, *, seed: int, max_num_sequence: Optional[int] = None,
              max_total_sequence_length: Optional[int] = None, prefill_chunk_size: Optional[int] = None,
              max_history_size: Optional[int] = None, gpu_memory_utilization: Optional[float] = None
              ) -> Dict[str, float]:
    """Run the calibration set and write the scales; returns ``{layer: absmax}``."""
    from ..serve.config import EngineConfig  # pylint: disable=import-outside-toplevel
    from ..serve.engine import MLCEngine  # pylint: disable=import-outside-toplevel

    random.seed(seed)
    # every matmul has to pass through ops.linear, eagerly: no captured graphs, no fused collectives
    saved = {k: os.environ.get(k) for k in ("MLCB_CUDA_GRAPH", "MLCB_FUSED_TP")}
    os.environ["MLCB_CUDA_GRAPH"] = "0"
    os.environ["MLCB_FUSED_TP"] = "0"
    observer = CalibrationObserver()
    try:
        engine = MLCEngine(model, device, model_lib=model_lib, mode="server",
                           engine_config=EngineConfig(max_num_sequence=max_num_sequence or 32,
                                                      max_total_sequence_length=max_total_sequence_length,
                                                      prefill_chunk_size=prefill_chunk_size,
                                                      max_history_size=max_history_size,
                                                      gpu_memory_utilization=gpu_memory_utilization))
        try:
            for m in engine.runtime.models:
                observer.watch(m)
            requests = sample_requests(dataset, num_calibration_samples, engine.tokenizer)
            ops.set_linear_observer(observer)
            for prompt, _, output_len in requests:
                engine.chat.completions.create(messages=[{"role": "user", "content": prompt}],
                                               max_tokens=output_len)
        finally:
            ops.set_linear_observer(None)
            engine.terminate()
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    observer.save_params(output)
    return {n: float(v.item()) for n, v in observer.params.items()}
