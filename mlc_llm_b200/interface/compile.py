"""``compile``: the reference lowers a model to a device library here (``interface/compile.py``).
This framework ships prebuilt sm_100a kernels and a config-driven model, so "compiling" a model means
checking that the architecture / quantisation / parallel layout is runnable and recording the
metadata the reference embeds in its libraries (``_metadata`` function: model type, quantisation,
window sizes, shard counts, parameter list, KV-cache layout, memory estimate).  The result is a small
JSON "model library" that ``--model-lib`` accepts."""

from __future__ import annotations

import json
import os
from typing import Dict, Optional

from .. import quantization as Q
from ..models import config as model_config
from ..models.transformer import param_specs
from ..support.auto_config import detect_config, detect_model_type


def model_metadata(cfg: model_config.ModelConfig, quant: Q.Quantization) -> Dict:
    specs = param_specs(cfg)
    params = []
    total = 0.0
    for name, (shape, kind) in specs.items():
        n = 1
        for s in shape:
            n *= s
        quantised = quant.kind != "no-quant" and kind in ("linear", "experts", "embedding")
        bits = (quant.bits + (16.0 / quant.group_size if quant.group_size else 0.0)) if quantised else (32 if quant.torch_dtype.itemsize == 4 else 16)
        total += n * bits / 8.0
        params.append({"name": name, "shape": list(shape), "kind": kind,
                       "dtype": quant.name if quantised else str(quant.torch_dtype).replace("torch.", "")})
    return {
        "model_type": cfg.model_type, "quantization": quant.name,
        "context_window_size": cfg.context_window_size, "sliding_window_size": cfg.sliding_window_size,
        "attention_sink_size": cfg.attention_sink_size, "prefill_chunk_size": cfg.prefill_chunk_size,
        "max_batch_size": cfg.max_batch_size, "tensor_parallel_shards": cfg.tensor_parallel_shards,
        "pipeline_parallel_stages": cfg.pipeline_parallel_stages,
        "kv_state_kind": "rnn_state" if cfg.extra.get("rwkv") else (
            "hybrid" if cfg.extra.get("gdn") else ("none" if cfg.extra.get("medusa") else "kv_cache")),
        "kv_cache": cfg.kv_cache_metadata(),
        "params": params, "memory_usage": {"params_bytes": total},
        "target": "sm_100a", "library": "libmlcb200_kernels.so",
    }


def compile_model(config: str, quantization: str, model_type: str = "auto", device: str = "cuda",
                  opt: Optional[str] = None, overrides: Optional[Dict] = None, output: str = "model-lib.json"
                  ) -> str:
    if device.split(":")[0] not in ("cuda", "auto", "cpu"):
        raise ValueError(f"target {device!r} is unavailable in this build (sm_100a CUDA only)")
    _, hf = detect_config(config)
    mt = detect_model_type(model_type, hf)
    merged = dict(hf)
    merged.update({k: v for k, v in (overrides or {}).items() if v is not None})
    cfg = model_config.from_dict(mt, merged)
    quant = Q.get(quantization)
    tp = max(1, cfg.tensor_parallel_shards)
    if cfg.num_key_value_heads % tp and tp % cfg.num_key_value_heads:
        raise ValueError("tensor_parallel_shards must divide (or be a multiple of) the KV head count")
    from .. import build  # pylint: disable=import-outside-toplevel

    meta = model_metadata(cfg, quant)
    meta["opt"] = opt or "O2"
    meta["kernels_built"] = os.path.exists(build.kernels_lib_path())
    os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
    with open(output, "w", encoding="utf-8") as f:
        json.dump(meta, f, indent=2)
    return output
