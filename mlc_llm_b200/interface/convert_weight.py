"""``convert_weight``: HuggingFace checkpoint -> quantised tensor cache (reference:
``python/mlc_llm/interface/convert_weight.py:32-216``).  Tensors are renamed / fused, quantised one
at a time on ``device`` (the GPU when present) and streamed into ``params_shard_*.bin``."""

from __future__ import annotations

import os
from typing import Optional

import torch

from .. import quantization as Q
from ..loader import huggingface_loader
from ..loader.tensor_cache import dump_tensor_cache
from ..models import config as model_config
from ..models.loader import export_params
from ..support.auto_config import detect_config, detect_device, detect_model_type, detect_weight


def convert_weight(config: str, quantization: str, model_type: str = "auto", device: str = "auto",
                   source: str = "auto", source_format: str = "auto", output: str = ".",
                   lora_adapter: Optional[str] = None, verbose: bool = True,
                   encode_format: str = "f32-to-bf16", preshard: int = 0) -> dict:
    """``preshard`` > 1 (or ``MLC_INTERNAL_PRESHARD_NUM``) writes every tensor-parallel parameter once per
    rank, already cut and quantised, as ``<name>_shard-<rank>`` (reference: ``support/preshard.py:16-17``);
    replicated parameters are written once. Ranks then read their own records without slicing."""
    config_path, hf = detect_config(config)
    mt = detect_model_type(model_type, hf)
    quant = Q.get(quantization)
    cfg = model_config.from_dict(mt, hf)
    dev = detect_device(device)
    src_dir, _fmt = detect_weight(source, config_path, source_format)
    os.makedirs(output, exist_ok=True)
    stats = {"params": 0, "bytes": 0}

    def on_device():
        for name, t in huggingface_loader.iter_mlc_params(src_dir, cfg, lora_adapter):
            yield name, t.to(dev)

    shards = int(preshard or os.environ.get("MLC_INTERNAL_PRESHARD_NUM", 0) or 0)

    def exported():
        if shards <= 1:
            yield from export_params(cfg, quant, on_device())
            return
        from ..models.loader import _shard_dense  # pylint: disable=import-outside-toplevel
        from ..models.transformer import param_specs  # pylint: disable=import-outside-toplevel

        specs = param_specs(cfg)
        ep = cfg.expert_parallel
        for name, w in on_device():
            kind = specs.get(name, (None, "norm"))[1]
            cuts = [_shard_dense(name, w, kind, cfg, shards, r, ep) for r in range(shards)]
            if all(c is w for c in cuts):
                yield from export_params(cfg, quant, iter([(name, w)]))
                continue
            for r, cut in enumerate(cuts):
                for out_name, t in export_params(cfg, quant, iter([(name, cut)])):
                    yield f"{out_name}_shard-{r}", t

    def records():
        for name, t in exported():
            t = t.cpu()
            stats["bytes"] += t.numel() * t.element_size()
            plain = name.split("_shard-")[0]
            if not (plain.endswith("q_scale") or plain.endswith("weight_scale_inv")):
                per_word = 32 // quant.bits if plain.endswith("q_weight") and quant.kind == "group-quant" else 1
                stats["params"] += t.numel() * per_word
            if verbose:
                print(f"[convert_weight] {name} {tuple(t.shape)} {t.dtype}")
            yield name, t
        if cfg.extra.get("vision"):
            # the vision tower and projector stay unquantised, under their checkpoint names
            from ..models.vision import load_hf_vision_params  # pylint: disable=import-outside-toplevel

            for name, t in load_hf_vision_params(src_dir, cfg.extra["vision"], cfg.hidden_size).items():
                t = t.to(torch.float32 if quant.torch_dtype == torch.float32 else torch.float16)
                stats["bytes"] += t.numel() * t.element_size()
                stats["params"] += t.numel()
                yield name, t

    doc = dump_tensor_cache(records(), output, encode_format=encode_format)
    total_params, total_bytes = stats["params"], stats["bytes"]
    bits = total_bytes * 8.0 / max(1, total_params)
    doc["metadata"].update({"ParamSize": sum(len(s["records"]) for s in doc["records"]),
                            "ParamBytes": float(total_bytes), "BitsPerParam": bits})
    import json  # pylint: disable=import-outside-toplevel

    with open(os.path.join(output, "tensor-cache.json"), "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=2)
    if verbose:
        print(f"[convert_weight] {total_params / 1e9:.3f} B parameters, {total_bytes / 2**30:.3f} GiB, "
              f"{bits:.3f} bits per parameter -> {output}")
    _ = torch
    return {"params": total_params, "bytes": total_bytes, "bits_per_param": bits}
