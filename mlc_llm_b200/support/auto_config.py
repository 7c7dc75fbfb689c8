"""Locate ``config.json`` / weights / model type / device from loosely specified CLI arguments
(reference: ``python/mlc_llm/support/auto_config.py``, ``auto_weight.py``, ``auto_device.py``)."""

from __future__ import annotations

import json
import os
from typing import Optional, Tuple

import torch

from ..models.config import SUPPORTED_MODEL_TYPES
from ..models.presets import MODEL_PRESETS


def detect_config(config: str) -> Tuple[str, dict]:
    """``config`` may be a preset name, a directory holding ``config.json`` or a JSON file. Returns
    (path or "preset:<name>", dict)."""
    if config in MODEL_PRESETS:
        return f"preset:{config}", dict(MODEL_PRESETS[config])
    path = config
    if os.path.isdir(path):
        for name in ("config.json", "mlc-chat-config.json"):
            if os.path.isfile(os.path.join(path, name)):
                path = os.path.join(path, name)
                break
        else:
            raise ValueError(f"{config}: no config.json in this directory")
    if not os.path.isfile(path):
        raise ValueError(f"{config}: not a preset name, a directory or a JSON file")
    with open(path, encoding="utf-8") as f:
        d = json.load(f)
    if "model_config" in d and "model_type" in d:  # an mlc-chat-config.json
        inner = dict(d["model_config"])
        inner.setdefault("model_type", d["model_type"])
        d = inner
    # multimodal wrappers keep the language model under text_config
    # (families whose parser reads the wrapper itself -- it also carries their vision section -- keep it)
    if "text_config" in d and isinstance(d["text_config"], dict) and "hidden_size" not in d \
            and d.get("model_type") not in ("llava", "llama4", "qwen3_5", "qwen2_5_vl"):
        merged = dict(d["text_config"])
        merged.setdefault("model_type", d.get("model_type"))
        d = merged
    return path, d


def detect_model_type(model_type: str, config: dict) -> str:
    if model_type != "auto":
        if model_type not in SUPPORTED_MODEL_TYPES:
            raise ValueError(f"unknown model type {model_type!r}; supported: {SUPPORTED_MODEL_TYPES}")
        return model_type
    mt = config.get("model_type")
    if mt is None:
        raise ValueError("config.json has no model_type; pass --model-type")
    mt = {"gemma3_text": "gemma3", "phi-msft": "phi", "stablelm_epoch": "stablelm"}.get(mt, mt)
    if mt not in SUPPORTED_MODEL_TYPES:
        raise ValueError(f"unsupported model type {mt!r}; supported: {SUPPORTED_MODEL_TYPES}")
    return mt


def detect_weight(source: str, config_path: str, source_format: str = "auto") -> Tuple[str, str]:
    """Returns (checkpoint directory, format in {"huggingface-safetensor", "huggingface-torch"})."""
    path = source
    if source == "auto":
        path = os.path.dirname(config_path)
    if os.path.isfile(path):
        path = os.path.dirname(path)
    has_st = any(f.endswith(".safetensors") for f in os.listdir(path))
    has_pt = any(f.endswith(".bin") and f.startswith("pytorch_model") for f in os.listdir(path))
    if source_format == "auto":
        if has_st:
            return path, "huggingface-safetensor"
        if has_pt:
            return path, "huggingface-torch"
        raise ValueError(f"no HuggingFace weights found under {path}")
    if source_format == "huggingface-safetensor" and not has_st:
        raise ValueError(f"no *.safetensors under {path}")
    if source_format == "huggingface-torch" and not has_pt:
        raise ValueError(f"no pytorch_model*.bin under {path}")
    if source_format == "awq":
        # AutoAWQ checkpoints are safetensors (or torch) files whose linear layers are (qweight, qzeros, scales)
        # triples: the HuggingFace reader expands them (loader/huggingface_loader.py), so only the container matters
        if has_st:
            return path, "huggingface-safetensor"
        if has_pt:
            return path, "huggingface-torch"
        raise ValueError(f"no AWQ weights (*.safetensors or pytorch_model*.bin) under {path}")
    return path, source_format


def detect_device(device: str) -> torch.device:
    """``auto`` prefers CUDA; ``cuda:N`` / ``cpu`` are taken literally. Graphics-API device names of
    other back ends (vulkan, metal, opencl, webgpu) are rejected."""
    if device == "auto":
        return torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    kind = device.split(":")[0]
    if kind not in ("cuda", "cpu"):
        raise ValueError(f"device {device!r} is not available in this build (cuda and cpu only)")
    return torch.device(device)
