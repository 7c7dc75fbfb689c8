"""Command line of ``mlc_llm_b200 serve`` (reference: ``python/mlc_llm/cli/serve.py:19-264``)."""

from __future__ import annotations

import argparse
import dataclasses
import json
from typing import Optional

from ..interface.serve import serve


@dataclasses.dataclass
class EngineConfigOverride:  # pylint: disable=too-many-instance-attributes
    """``--overrides "key=value;key=value"`` for the numeric engine options."""

    max_num_sequence: Optional[int] = None
    max_total_seq_length: Optional[int] = None
    max_single_sequence_length: Optional[int] = None
    prefill_chunk_size: Optional[int] = None
    sliding_window_size: Optional[int] = None
    attention_sink_size: Optional[int] = None
    max_history_size: Optional[int] = None
    gpu_memory_utilization: Optional[float] = None
    spec_draft_length: Optional[int] = None
    spec_tree_width: Optional[int] = None
    prefix_cache_max_num_recycling_seqs: Optional[int] = None
    tensor_parallel_shards: Optional[int] = None
    pipeline_parallel_stages: Optional[int] = None
    opt: Optional[str] = None

    @staticmethod
    def from_str(source: str) -> "EngineConfigOverride":
        out = EngineConfigOverride()
        fields = {f.name: f.type for f in dataclasses.fields(EngineConfigOverride)}
        aliases = {"max_total_sequence_length": "max_total_seq_length"}
        for item in filter(None, (part.strip() for part in source.split(";"))):
            if "=" not in item:
                raise argparse.ArgumentTypeError(f"override {item!r} is not of the form key=value")
            key, value = (x.strip() for x in item.split("=", 1))
            key = aliases.get(key, key)
            if key not in fields:
                raise argparse.ArgumentTypeError(f"unknown engine override {key!r}")
            if key == "opt":
                setattr(out, key, value)
            elif key == "gpu_memory_utilization":
                setattr(out, key, float(value))
            else:
                setattr(out, key, int(value))
        return out


def _additional_models(text: str):
    if "," in text:
        path, lib = text.split(",", 1)
        return (path, lib)
    return text


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("mlc_llm_b200 serve", description="Launch the OpenAI-compatible REST server")
    p.add_argument("model", type=str, help="model directory (with mlc-chat-config.json), or random://<preset>")
    p.add_argument("--device", type=str, default="auto")
    p.add_argument("--model-lib", type=str, default=None,
                   help="accepted for command-line compatibility; kernels are prebuilt (only mock://echo is honoured)")
    p.add_argument("--mode", type=str, choices=["local", "interactive", "server"], default="local")
    p.add_argument("--enable-debug", action="store_true")
    p.add_argument("--additional-models", type=_additional_models, nargs="*", default=[])
    p.add_argument("--embedding-model", type=str, default=None)
    p.add_argument("--embedding-model-lib", type=str, default=None)
    p.add_argument("--speculative-mode", type=str, choices=["disable", "small_draft", "eagle", "medusa"],
                   default="disable")
    p.add_argument("--prefix-cache-mode", type=str, choices=["disable", "radix"], default="radix")
    p.add_argument("--prefill-mode", type=str, choices=["hybrid", "chunked"], default="hybrid")
    p.add_argument("--overrides", type=EngineConfigOverride.from_str, default="")
    p.add_argument("--enable-tracing", action="store_true")
    p.add_argument("--host", type=str, default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--allow-credentials", action="store_true")
    p.add_argument("--allow-origins", type=json.loads, default=["*"])
    p.add_argument("--allow-methods", type=json.loads, default=["*"])
    p.add_argument("--allow-headers", type=json.loads, default=["*"])
    p.add_argument("--api-key", type=str, default=None)
    return p


def main(argv=None) -> None:
    args = build_parser().parse_args(argv)
    ov = args.overrides if isinstance(args.overrides, EngineConfigOverride) else EngineConfigOverride()
    serve(model=args.model, device=args.device, model_lib=args.model_lib, mode=args.mode,
          enable_debug=args.enable_debug, additional_models=args.additional_models,
          embedding_model=args.embedding_model, embedding_model_lib=args.embedding_model_lib,
          tensor_parallel_shards=ov.tensor_parallel_shards, pipeline_parallel_stages=ov.pipeline_parallel_stages,
          opt=ov.opt, max_num_sequence=ov.max_num_sequence, max_total_sequence_length=ov.max_total_seq_length,
          max_single_sequence_length=ov.max_single_sequence_length, prefill_chunk_size=ov.prefill_chunk_size,
          sliding_window_size=ov.sliding_window_size, attention_sink_size=ov.attention_sink_size,
          max_history_size=ov.max_history_size, gpu_memory_utilization=ov.gpu_memory_utilization,
          speculative_mode=args.speculative_mode, spec_draft_length=ov.spec_draft_length,
          spec_tree_width=ov.spec_tree_width, prefix_cache_mode=args.prefix_cache_mode,
          prefix_cache_max_num_recycling_seqs=ov.prefix_cache_max_num_recycling_seqs,
          prefill_mode=args.prefill_mode, enable_tracing=args.enable_tracing, host=args.host, port=args.port,
          allow_credentials=args.allow_credentials, allow_origins=args.allow_origins,
          allow_methods=args.allow_methods, allow_headers=args.allow_headers, api_key=args.api_key)


if __name__ == "__main__":
    main()
