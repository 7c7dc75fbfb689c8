"""Python ``EngineConfig`` (JSON round-trip with the native config; reference
``python/mlc_llm/serve/config.py:8-169`` and ``cpp/serve/config.h:236-324``)."""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import List, Literal, Optional, Tuple, Union


@dataclass
class EngineConfig:  # pylint: disable=too-many-instance-attributes
    """Engine options. Everything left ``None`` is inferred at start-up from the mode, the model and
    the GPU memory budget (see ``_core.infer_capacity``)."""

    model: Optional[str] = None
    model_lib: Optional[str] = None
    additional_models: List[Union[str, Tuple[str, str]]] = field(default_factory=list)
    mode: Optional[Literal["local", "interactive", "server"]] = None
    tensor_parallel_shards: Optional[int] = None
    pipeline_parallel_stages: Optional[int] = None
    opt: Optional[str] = None
    gpu_memory_utilization: Optional[float] = None
    kv_cache_page_size: int = 16
    max_num_sequence: Optional[int] = None
    max_total_sequence_length: Optional[int] = None
    max_single_sequence_length: Optional[int] = None
    prefill_chunk_size: Optional[int] = None
    sliding_window_size: Optional[int] = None
    attention_sink_size: Optional[int] = None
    max_history_size: Optional[int] = None
    kv_state_kind: Optional[Literal["kv_cache", "rnn_state", "hybrid"]] = None
    speculative_mode: Literal["disable", "small_draft", "eagle", "medusa"] = "disable"
    spec_draft_length: int = 0
    spec_tree_width: int = 1
    prefix_cache_mode: Literal["disable", "radix"] = "radix"
    prefix_cache_max_num_recycling_seqs: Optional[int] = None
    prefill_mode: Literal["chunked", "hybrid"] = "hybrid"
    verbose: bool = True

    def asjson(self) -> str:
        d = {k: v for k, v in asdict(self).items() if v is not None}
        return json.dumps(d)

    @staticmethod
    def from_json(json_str: str) -> "EngineConfig":
        d = json.loads(json_str)
        known = EngineConfig.__dataclass_fields__  # pylint: disable=no-member
        clean = {}
        for k, v in d.items():
            if k not in known:
                continue
            # the native side writes -1 for "unset"
            if isinstance(v, int) and not isinstance(v, bool) and v == -1 and k not in ("spec_draft_length",):
                v = None
            if v == "" and k in ("model_lib", "opt", "model"):
                v = None
            clean[k] = v
        return EngineConfig(**clean)
