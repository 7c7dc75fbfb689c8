"""``gen_config``: write ``mlc-chat-config.json`` and copy the tokenizer files (reference:
``python/mlc_llm/interface/gen_config.py:88-300``)."""

from __future__ import annotations

import json
import os
import shutil
from typing import Optional

from .. import quantization as Q
from ..conversation_template import ConvTemplateRegistry
from ..models import config as model_config
from ..protocol.mlc_chat_config import MLCChatConfig
from ..support.auto_config import detect_config, detect_model_type

TOKENIZER_FILES = ["tokenizer.model", "tokenizer.json", "vocab.json", "merges.txt", "added_tokens.json",
                   "tokenizer_config.json", "tokenizer_model"]

CONV_TEMPLATES = set(ConvTemplateRegistry.names())


def gen_config(config: str, model_type: str, quantization: str, conv_template: str,  # pylint: disable=too-many-arguments,too-many-locals
               context_window_size: Optional[int], sliding_window_size: Optional[int],
               prefill_chunk_size: Optional[int], attention_sink_size: Optional[int],
               tensor_parallel_shards: Optional[int], pipeline_parallel_stages: Optional[int],
               disaggregation: Optional[bool], max_batch_size: int, output: str) -> str:
    config_path, hf = detect_config(config)
    mt = detect_model_type(model_type, hf)
    quant = Q.get(quantization)
    conv = ConvTemplateRegistry.get_conv_template(conv_template)
    if conv is None:
        raise ValueError(f"conversation template {conv_template!r} is not registered; known: "
                         f"{sorted(CONV_TEMPLATES)}")
    overrides = {"context_window_size": context_window_size, "sliding_window_size": sliding_window_size,
                 "prefill_chunk_size": prefill_chunk_size, "attention_sink_size": attention_sink_size,
                 "tensor_parallel_shards": tensor_parallel_shards,
                 "pipeline_parallel_stages": pipeline_parallel_stages, "max_batch_size": max_batch_size}
    merged = dict(hf)
    merged.update({k: v for k, v in overrides.items() if v is not None})
    cfg = model_config.from_dict(mt, merged)
    if cfg.sliding_window_size and cfg.sliding_window_size > 0:
        cfg.context_window_size = -1
    # the checkpoint's own keys stay in the model section (family parsers read settings such as expert
    # routing, latent-attention ranks, recurrent-layer geometry or a nested text / vision config from
    # them when the engine parses the section again); resolved structural fields are written over them
    resolved = cfg.asdict()
    mc = {k: v for k, v in merged.items() if k not in ("architectures", "torch_dtype", "dtype", "transformers_version",
                                                        "id2label", "label2id", "auto_map")}
    for k, v in resolved.items():
        if k not in mc or k in overrides or k in ("context_window_size", "sliding_window_size",
                                                  "prefill_chunk_size", "attention_sink_size"):
            mc[k] = v
    if disaggregation:
        mc["disaggregation"] = True
    os.makedirs(output, exist_ok=True)
    chat = MLCChatConfig(
        model_type=mt, quantization=quant.name, model_config=mc, vocab_size=cfg.vocab_size,
        active_vocab_size=cfg.vocab_size, context_window_size=cfg.context_window_size,
        sliding_window_size=cfg.sliding_window_size, prefill_chunk_size=cfg.prefill_chunk_size,
        attention_sink_size=cfg.attention_sink_size, tensor_parallel_shards=cfg.tensor_parallel_shards,
        pipeline_parallel_stages=cfg.pipeline_parallel_stages, conv_template=conv,
        model_task="embedding" if mt == "bert" else "chat")
    src_dir = os.path.dirname(config_path) if not config_path.startswith("preset:") else None
    if src_dir is not None:
        for name in ("generation_config.json", "config.json"):
            p = os.path.join(src_dir, name)
            if not os.path.isfile(p):
                continue
            with open(p, encoding="utf-8") as f:
                gen = json.load(f)
            for key, value in gen.items():
                if key in MLCChatConfig.model_fields and getattr(chat, key, None) is None:
                    setattr(chat, key, value)
        for name in TOKENIZER_FILES:
            p = os.path.join(src_dir, name)
            if os.path.isfile(p):
                chat.tokenizer_files.append(name)
                if os.path.abspath(p) != os.path.abspath(os.path.join(output, name)):
                    shutil.copy(p, os.path.join(output, name))
        if "tokenizer.model" in chat.tokenizer_files and "tokenizer.json" not in chat.tokenizer_files:
            try:  # prefer the JSON form (same attempt as the reference makes)
                from transformers import AutoTokenizer  # pylint: disable=import-outside-toplevel

                AutoTokenizer.from_pretrained(src_dir, use_fast=True).backend_tokenizer.save(
                    os.path.join(output, "tokenizer.json"))
                chat.tokenizer_files.append("tokenizer.json")
            except Exception:  # pylint: disable=broad-except
                pass
        if not chat.tokenizer_files and any(f.endswith(".tiktoken") for f in os.listdir(src_dir)):
            # tiktoken rank file (first-generation Qwen and others): converted once to the HuggingFace form
            from ..support.convert_tiktoken import convert_tiktoken  # pylint: disable=import-outside-toplevel

            convert_tiktoken(src_dir, output)
            chat.tokenizer_files.extend(["tokenizer.json", "vocab.json", "merges.txt"])
        if chat.tokenizer_files:
            from ..tokenizers import Tokenizer  # pylint: disable=import-outside-toplevel

            try:
                chat.tokenizer_info = Tokenizer.detect_tokenizer_info(output)
            except Exception:  # pylint: disable=broad-except
                chat.tokenizer_info = {}
    chat.apply_system_defaults()
    out_path = os.path.join(output, "mlc-chat-config.json")
    with open(out_path, "w", encoding="utf-8") as f:
        json.dump(chat.model_dump(by_alias=True), f, indent=2)
    return out_path
