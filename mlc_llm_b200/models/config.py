"""Normalised architecture description shared by every decoder family.

Each supported ``model_type`` maps its HuggingFace / mlc-chat-config fields onto one
``ModelConfig``; the generic decoder in ``models/transformer.py`` is driven entirely by it.
Reference: the per-family config classes under ``python/mlc_llm/model/*/`` (canonical one:
``model/llama/llama_model.py:24-103``) and the registry ``model/model.py:134+``.
"""

from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, List, Optional


@dataclasses.dataclass
class ModelConfig:
    model_type: str = "llama"
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 0
    head_dim: int = 0
    vocab_size: int = 32000
    rms_norm_eps: float = 1e-5
    # positions
    position_embedding: str = "rope"  # "rope" | "learned" | "none"
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    partial_rotary_factor: float = 1.0
    max_position_embeddings: int = 0
    # sizes the runtime cares about
    context_window_size: int = 0
    prefill_chunk_size: int = 0
    sliding_window_size: int = -1
    attention_sink_size: int = -1
    tensor_parallel_shards: int = 1
    pipeline_parallel_stages: int = 1
    max_batch_size: int = 128
    # structure switches
    norm_type: str = "rms"              # "rms" | "layernorm"
    norm_weight_offset: float = 0.0     # gemma stores (w - 1)
    hidden_act: str = "silu"            # "silu" | "gelu_tanh" | "gelu" | "relu2"
    gated_mlp: bool = True
    attention_bias: bool = False        # bias on q/k/v
    attention_out_bias: bool = False
    mlp_bias: bool = False
    qk_norm: bool = False               # per-head RMSNorm on q and k (qwen3, olmo2, gemma3)
    tie_word_embeddings: bool = False
    embedding_scale: float = 1.0        # gemma multiplies embeddings by sqrt(hidden)
    parallel_residual: bool = False     # gpt-neox / phi-2 style x + attn(ln(x)) + mlp(ln(x))
    shared_input_norm: bool = False     # with parallel_residual: one norm feeds both branches
    post_attention_norm: bool = False   # gemma2/3: extra norms after attention and after the MLP
    post_mlp_norm: bool = False
    query_pre_attn_scalar: float = 0.0  # gemma2: sm_scale = this ** -0.5
    attn_logit_softcap: float = 0.0
    final_logit_softcap: float = 0.0
    layer_attn_kinds: Optional[List[str]] = None  # per-layer "mha" | "mha_sliding"
    rope_local_theta: float = 0.0       # gemma3: theta of sliding layers
    lm_head_bias: bool = False
    # mixture of experts
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    moe_router: str = "topk_softmax"    # "topk_softmax" (mixtral) | "softmax_topk" (qwen-moe)
    shared_expert_intermediate_size: int = 0
    shared_expert_gate: bool = False
    moe_layer_freq: int = 1
    first_moe_layer: int = 0
    expert_parallel: bool = False       # shard experts across ranks instead of their width
    extra: Dict[str, Any] = dataclasses.field(default_factory=dict)

    def __post_init__(self):
        if self.num_key_value_heads <= 0:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim <= 0:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.context_window_size <= 0:
            self.context_window_size = self.max_position_embeddings or 8192
        if self.prefill_chunk_size <= 0:
            self.prefill_chunk_size = min(self.context_window_size, 8192)
        if self.moe_intermediate_size <= 0 and self.num_experts > 0:
            self.moe_intermediate_size = self.intermediate_size

    @property
    def rotary_dim(self) -> int:
        r = int(self.head_dim * self.partial_rotary_factor)
        return r - (r % 2)

    def is_moe_layer(self, layer: int) -> bool:
        # Qwen counts sparse layers as (layer + 1) % step == 0, DeepSeek as layer % freq == 0
        if "moe_layers" in self.extra:  # explicit list (Llama-4)
            return self.num_experts > 0 and layer in self.extra["moe_layers"]
        phase = int(self.extra.get("moe_layer_phase", 1))
        return (self.num_experts > 0 and layer >= self.first_moe_layer
                and (layer + phase) % max(1, self.moe_layer_freq) == 0)

    def kv_cache_metadata(self) -> Dict[str, int]:
        tp = max(1, self.tensor_parallel_shards)
        return {"num_hidden_layers": self.num_hidden_layers,
                "num_attention_heads": self.num_attention_heads // tp,
                "num_key_value_heads": max(1, self.num_key_value_heads // tp),
                "head_dim": self.head_dim}

    def asdict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        d.pop("extra")
        return d


def _get(cfg: Dict[str, Any], *names, default=None):
    for n in names:
        if n in cfg and cfg[n] is not None:
            return cfg[n]
    return default


def _common(cfg: Dict[str, Any], model_type: str) -> Dict[str, Any]:
    """Fields spelled the same way by most HuggingFace configs."""
    rp = cfg.get("rope_parameters")
    if isinstance(rp, dict):  # newer transformers nest the rotary settings
        cfg = dict(cfg)
        if "rope_theta" in rp and cfg.get("rope_theta") is None:
            cfg["rope_theta"] = rp["rope_theta"]
        if rp.get("rope_type", "default") != "default" and cfg.get("rope_scaling") is None:
            cfg["rope_scaling"] = {k: v for k, v in rp.items() if k != "rope_theta"}
        if "partial_rotary_factor" in rp and cfg.get("partial_rotary_factor") is None:
            cfg["partial_rotary_factor"] = rp["partial_rotary_factor"]
    if isinstance(cfg.get("rope_scaling"), dict):
        # stretched-context variants need the trained and the served window next to their factors
        rs = dict(cfg["rope_scaling"])
        for key in ("original_max_position_embeddings", "max_position_embeddings"):
            if rs.get(key) is None and cfg.get(key) is not None:
                rs[key] = cfg[key]
        cfg = dict(cfg, rope_scaling=rs)
    out = dict(
        model_type=model_type,
        hidden_size=_get(cfg, "hidden_size", "n_embd", "d_model", default=4096),
        intermediate_size=_get(cfg, "intermediate_size", "n_inner", "ffn_dim", default=0) or 0,
        num_hidden_layers=_get(cfg, "num_hidden_layers", "n_layer", "num_layers", default=32),
        num_attention_heads=_get(cfg, "num_attention_heads", "n_head", default=32),
        num_key_value_heads=_get(cfg, "num_key_value_heads", "num_kv_heads", default=0) or 0,
        head_dim=_get(cfg, "head_dim", default=0) or 0,
        vocab_size=_get(cfg, "vocab_size", default=32000),
        rms_norm_eps=_get(cfg, "rms_norm_eps", "layer_norm_eps", "layer_norm_epsilon", "norm_eps",
                          "norm_epsilon", default=1e-5),
        rope_theta=float(_get(cfg, "rope_theta", "position_embedding_base", "rotary_emb_base",
                              default=10000.0)),
        rope_scaling=_get(cfg, "rope_scaling"),
        max_position_embeddings=_get(cfg, "max_position_embeddings", "n_positions",
                                     "max_sequence_length", default=0) or 0,
        context_window_size=_get(cfg, "context_window_size", default=0) or 0,
        prefill_chunk_size=_get(cfg, "prefill_chunk_size", default=0) or 0,
        sliding_window_size=_get(cfg, "sliding_window_size", default=-1),
        attention_sink_size=_get(cfg, "attention_sink_size", default=-1),
        tensor_parallel_shards=_get(cfg, "tensor_parallel_shards", default=1),
        pipeline_parallel_stages=_get(cfg, "pipeline_parallel_stages", default=1),
        max_batch_size=_get(cfg, "max_batch_size", default=128),
        tie_word_embeddings=bool(_get(cfg, "tie_word_embeddings", default=False)),
    )
    if out["intermediate_size"] == 0:
        out["intermediate_size"] = 4 * out["hidden_size"]
    return out


def _llama(cfg, mt):
    d = _common(cfg, mt)
    d["attention_bias"] = bool(_get(cfg, "attention_bias", default=False))
    d["attention_out_bias"] = d["attention_bias"]
    d["mlp_bias"] = bool(_get(cfg, "mlp_bias", default=False))
    return d


def _llama4(cfg, mt):
    """Llama-4 text model: rotary layers with chunked attention and weightless q / k L2 norm, interleaved
    with position-free layers whose queries are scaled by a temperature that grows with the position;
    mixture-of-experts layers route on the top logit, scale the expert *input* by its sigmoid and add a shared
    expert (reference: ``python/mlc_llm/model/llama4/llama4_model.py``)."""
    if isinstance(cfg.get("text_config"), dict):
        outer, cfg = cfg, dict(cfg["text_config"])
        for k in ("context_window_size", "prefill_chunk_size", "tensor_parallel_shards", "max_batch_size"):
            if k in outer and k not in cfg:
                cfg[k] = outer[k]
    d = _llama(cfg, mt)
    layers = int(d["num_hidden_layers"])
    expert_inter = int(_get(cfg, "intermediate_size", default=8192))
    d["intermediate_size"] = int(_get(cfg, "intermediate_size_mlp", default=16384))
    use_rope = _get(cfg, "no_rope_layers") or [int((i + 1) % 4 != 0) for i in range(layers)]
    step = int(_get(cfg, "interleave_moe_layer_step", default=1))
    moe_layers = _get(cfg, "moe_layers")
    if moe_layers is None:
        moe_layers = list(range(step - 1, layers, step))
    chunk = int(_get(cfg, "attention_chunk_size", default=8192) or 0)
    d.update(num_experts=int(_get(cfg, "num_local_experts", default=16)),
             num_experts_per_tok=int(_get(cfg, "num_experts_per_tok", default=1)),
             moe_intermediate_size=expert_inter, shared_expert_intermediate_size=expert_inter,
             moe_router="llama4_sigmoid",
             layer_attn_kinds=["mha_chunked" if r else "mha_nope" for r in use_rope])
    d["extra"] = {"moe_layers": [int(x) for x in moe_layers],
                  "llama4": {"use_qk_norm": bool(_get(cfg, "use_qk_norm", default=True)),
                             "attn_temperature_tuning": bool(_get(cfg, "attn_temperature_tuning", default=True)),
                             "floor_scale": float(_get(cfg, "floor_scale", default=8192)),
                             "attn_scale": float(_get(cfg, "attn_scale", default=0.1)),
                             "attention_chunk_size": chunk}}
    return d


def _minicpm(cfg, mt):
    """MiniCPM: Llama blocks with scaled embeddings, residual branches scaled by
    ``scale_depth / sqrt(num_layers)`` and hidden states divided by ``hidden / dim_model_base`` before the
    head (reference: ``python/mlc_llm/model/minicpm/minicpm_model.py:300-314,355-372,386``)."""
    d = _llama(cfg, mt)
    layers = int(d["num_hidden_layers"])
    d["embedding_scale"] = float(_get(cfg, "scale_emb", default=1))
    width = max(1, int(d["hidden_size"]) // int(_get(cfg, "dim_model_base", default=d["hidden_size"])))
    d["extra"] = {"residual_scale": float(_get(cfg, "scale_depth", default=1.0)) / math.sqrt(layers),
                  "logit_scale": 1.0 / width}
    return d


def _internlm(cfg, mt):
    d = _llama(cfg, mt)
    if "bias" in cfg and "attention_bias" not in cfg:  # InternLM spells the q/k/v/o bias switch "bias"
        d["attention_bias"] = d["attention_out_bias"] = bool(cfg["bias"])
    return d


def _orion(cfg, mt):
    d = _llama(cfg, mt)
    d["norm_type"] = "layernorm"  # reference: python/mlc_llm/model/orion/orion_model.py:149-150,195
    return d


def _mistral(cfg, mt):
    d = _common(cfg, mt)
    sw = _get(cfg, "sliding_window")
    if sw and d["sliding_window_size"] in (-1, None) and not d["context_window_size"]:
        d["sliding_window_size"] = int(sw)
        d["attention_sink_size"] = max(0, d["attention_sink_size"] or 0) if d["attention_sink_size"] != -1 else 4
        d["context_window_size"] = -1 if False else 0
    return d


def _ministral3(cfg, mt):
    """Ministral 3: Mistral blocks under ``text_config``, YaRN rotary scaling, and queries multiplied by
    ``1 + beta * ln(1 + floor(position / trained window))`` (reference:
    ``python/mlc_llm/model/ministral3/ministral3_model.py``)."""
    if isinstance(cfg.get("text_config"), dict):
        outer, cfg = cfg, dict(cfg["text_config"])
        for k in ("context_window_size", "prefill_chunk_size", "sliding_window_size", "attention_sink_size",
                  "tensor_parallel_shards", "pipeline_parallel_stages", "max_batch_size"):
            if k in outer and k not in cfg:
                cfg[k] = outer[k]
    d = _mistral(cfg, mt)
    rp = cfg.get("rope_parameters") if isinstance(cfg.get("rope_parameters"), dict) else (cfg.get("rope_scaling") or {})
    beta = rp.get("llama_4_scaling_beta")
    if beta:
        d["extra"] = {"q_pos_scale": {"beta": float(beta),
                                      "window": int(rp.get("original_max_position_embeddings")
                                                    or cfg.get("max_position_embeddings") or 1)}}
    return d


def _qwen(cfg, mt):
    """Qwen (first generation): Llama math with a q/k/v bias; ``intermediate_size`` in its config counts
    gate and up together (reference: ``python/mlc_llm/model/qwen/qwen_model.py:118-134``)."""
    cfg = dict(cfg)
    if "kv_channels" in cfg and "head_dim" not in cfg:
        cfg["head_dim"] = cfg["kv_channels"]
    cfg.setdefault("rms_norm_eps", cfg.get("layer_norm_epsilon", 1e-6))
    cfg.setdefault("rope_theta", cfg.get("rotary_emb_base", 10000.0))
    cfg.setdefault("max_position_embeddings", cfg.get("seq_length", 8192))
    d = _common(cfg, mt)
    d["intermediate_size"] = int(d["intermediate_size"]) // 2
    d["attention_bias"] = True
    d["attention_out_bias"] = False
    return d


def _qwen2(cfg, mt):
    d = _common(cfg, mt)
    d["attention_bias"] = True
    return d


def _qwen3(cfg, mt):
    d = _common(cfg, mt)
    d["attention_bias"] = bool(_get(cfg, "attention_bias", default=False))
    d["qk_norm"] = True
    return d


def _gemma(cfg, mt):
    d = _common(cfg, mt)
    d["norm_weight_offset"] = 1.0
    d["hidden_act"] = "gelu_tanh"
    d["embedding_scale"] = math.sqrt(d["hidden_size"])
    d["tie_word_embeddings"] = True
    if mt in ("gemma2", "gemma3", "gemma3_text"):
        d["post_attention_norm"] = True
        d["post_mlp_norm"] = True
        d["query_pre_attn_scalar"] = float(_get(cfg, "query_pre_attn_scalar", default=0) or 0)
        d["attn_logit_softcap"] = float(_get(cfg, "attn_logit_softcapping", default=0) or 0)
        d["final_logit_softcap"] = float(_get(cfg, "final_logit_softcapping", default=0) or 0)
        sw = _get(cfg, "sliding_window", default=4096)
        n = d["num_hidden_layers"]
        if mt == "gemma2":
            d["layer_attn_kinds"] = ["mha_sliding" if i % 2 == 0 else "mha" for i in range(n)]
        else:
            pat = _get(cfg, "sliding_window_pattern", default=6)
            d["layer_attn_kinds"] = ["mha" if (i + 1) % pat == 0 else "mha_sliding" for i in range(n)]
            d["qk_norm"] = True
            d["rope_local_theta"] = float(_get(cfg, "rope_local_base_freq", default=10000.0))
        d["extra"] = {"layer_sliding_window": int(sw)}
    return d


def _phi3(cfg, mt):
    d = _common(cfg, mt)
    return d


def _phi(cfg, mt):
    d = _common(cfg, mt)
    d.update(norm_type="layernorm", hidden_act="gelu_tanh", gated_mlp=False, attention_bias=True,
             attention_out_bias=True, mlp_bias=True, parallel_residual=True, shared_input_norm=True,
             partial_rotary_factor=float(_get(cfg, "partial_rotary_factor", default=0.4)),
             lm_head_bias=True)
    return d


def _gpt_neox(cfg, mt):
    d = _common(cfg, mt)
    d.update(norm_type="layernorm", hidden_act="gelu", gated_mlp=False, attention_bias=True,
             attention_out_bias=True, mlp_bias=True,
             parallel_residual=bool(_get(cfg, "use_parallel_residual", default=True)),
             partial_rotary_factor=float(_get(cfg, "rotary_pct", default=0.25)))
    return d


def _gptj(cfg, mt):
    """GPT-J: one LayerNorm feeds attention and MLP in parallel, rotary embedding on the first
    ``rotary_dim`` dimensions of every head (reference: ``python/mlc_llm/model/gpt_j/gpt_j_model.py``).
    The checkpoint's interleaved rotary layout is converted to the half-split one when weights load."""
    d = _common(cfg, mt)
    head_dim = d["hidden_size"] // d["num_attention_heads"]
    rot = int(_get(cfg, "rotary_dim", default=head_dim) or head_dim)
    d.update(norm_type="layernorm", hidden_act="gelu_tanh", gated_mlp=False, attention_bias=False,
             attention_out_bias=False, mlp_bias=True, parallel_residual=True, shared_input_norm=True,
             partial_rotary_factor=rot / head_dim, lm_head_bias=True, tie_word_embeddings=False)
    return d


def _glm(cfg, mt):
    """GLM-4 (HuggingFace ``glm``) and ChatGLM3: RMSNorm Llama-style blocks with q/k/v bias and rotary
    embedding on the first half of every head, stored interleaved in the checkpoint (reference:
    ``python/mlc_llm/model/chatglm3/chatglm3_model.py``)."""
    if mt == "chatglm":
        cfg = dict(cfg)
        ren = {"num_layers": "num_hidden_layers", "multi_query_group_num": "num_key_value_heads",
               "kv_channels": "head_dim", "ffn_hidden_size": "intermediate_size",
               "layernorm_epsilon": "rms_norm_eps", "padded_vocab_size": "vocab_size",
               "seq_length": "max_position_embeddings"}
        for old, new in ren.items():
            if old in cfg and new not in cfg:
                cfg[new] = cfg[old]
        if not cfg.get("multi_query_attention", True):
            cfg["num_key_value_heads"] = cfg["num_attention_heads"]
        cfg.setdefault("rope_theta", 10000.0 * float(cfg.get("rope_ratio", 1.0)))
        cfg.setdefault("attention_bias", bool(cfg.get("add_qkv_bias", True)))
    d = _common(cfg, mt)
    d["attention_bias"] = bool(_get(cfg, "attention_bias", default=True))
    d["attention_out_bias"] = False
    d["partial_rotary_factor"] = float(_get(cfg, "partial_rotary_factor", default=0.5))
    d["extra"] = {"rope_interleaved_in_checkpoint": True}
    return d


def _rwkv5(cfg, mt):
    """RWKV-5: recurrent blocks, no attention (reference: ``python/mlc_llm/model/rwkv5/rwkv5_model.py``)."""
    hidden = int(_get(cfg, "hidden_size"))
    head = int(_get(cfg, "head_size", default=64))
    inter = _get(cfg, "intermediate_size")
    if not inter:
        inter = int((hidden * 3.5)) // 32 * 32
    return dict(model_type=mt, hidden_size=hidden, intermediate_size=int(inter),
                num_hidden_layers=int(_get(cfg, "num_hidden_layers")), num_attention_heads=hidden // head,
                num_key_value_heads=hidden // head, head_dim=head, vocab_size=int(_get(cfg, "vocab_size")),
                rms_norm_eps=float(_get(cfg, "layer_norm_epsilon", default=1e-5)), norm_type="layernorm",
                position_embedding="none", context_window_size=int(_get(cfg, "context_window_size", default=0) or 0) or -1,
                prefill_chunk_size=int(_get(cfg, "prefill_chunk_size", default=0) or 0),
                max_batch_size=int(_get(cfg, "max_batch_size", default=128)),
                extra={"rwkv": 6 if mt == "rwkv6" else 5,
                       "rescale_every": int(_get(cfg, "rescale_every", default=0) or 0),
                       # widths of RWKV-6's low-rank corrections (reference: rwkv6_model.py:203-209)
                       "time_mix_extra_dim": 64 if hidden == 4096 else 32,
                       "time_decay_extra_dim": 128 if hidden == 4096 else 64})


def _gpt2(cfg, mt):
    d = _common(cfg, mt)
    d.update(norm_type="layernorm", hidden_act="gelu_tanh", gated_mlp=False, attention_bias=True,
             attention_out_bias=True, mlp_bias=True, position_embedding="learned",
             tie_word_embeddings=True)
    if mt == "gpt_bigcode":
        d["num_key_value_heads"] = 1 if _get(cfg, "multi_query", default=True) else 0
    return d


def _starcoder2(cfg, mt):
    d = _common(cfg, mt)
    d.update(norm_type="layernorm", hidden_act="gelu_tanh", gated_mlp=False, attention_bias=True,
             attention_out_bias=True, mlp_bias=True)
    return d


def _stablelm(cfg, mt):
    d = _common(cfg, mt)
    d.update(norm_type="layernorm", attention_bias=bool(_get(cfg, "use_qkv_bias", default=False)),
             partial_rotary_factor=float(_get(cfg, "partial_rotary_factor", "rope_pct", default=0.25)))
    return d


def _olmo(cfg, mt):
    d = _common(cfg, mt)
    if mt == "olmo2":
        d["qk_norm"] = True
        d["post_attention_norm"] = True
        d["post_mlp_norm"] = True
        d["extra"] = {"no_pre_norm": True, "qk_norm_full": True}
    else:
        d["norm_type"] = "layernorm"
        d["extra"] = {"norm_no_affine": True}
    return d


def _mixtral(cfg, mt):
    d = _common(cfg, mt)
    d.update(num_experts=_get(cfg, "num_local_experts", "num_experts", default=8),
             num_experts_per_tok=_get(cfg, "num_experts_per_tok", default=2),
             moe_router="topk_softmax", expert_parallel=bool(_get(cfg, "expert_parallel", default=False)))
    d["moe_intermediate_size"] = d["intermediate_size"]
    return d


def _qwen_moe(cfg, mt):
    d = _common(cfg, mt)
    d.update(num_experts=_get(cfg, "num_experts", "num_local_experts", default=60),
             num_experts_per_tok=_get(cfg, "num_experts_per_tok", default=4),
             moe_intermediate_size=_get(cfg, "moe_intermediate_size", default=1408),
             norm_topk_prob=bool(_get(cfg, "norm_topk_prob", default=False)),
             moe_router="softmax_topk",
             shared_expert_intermediate_size=_get(cfg, "shared_expert_intermediate_size", default=0) or 0,
             moe_layer_freq=_get(cfg, "decoder_sparse_step", default=1),
             expert_parallel=bool(_get(cfg, "expert_parallel", default=False)))
    if mt == "qwen2_moe":
        d["attention_bias"] = True
        d["shared_expert_gate"] = True
    else:
        d["qk_norm"] = True
    return d


def _deepseek_moe_fields(cfg, d):
    routed = int(_get(cfg, "n_routed_experts", default=0) or 0)
    shared = int(_get(cfg, "n_shared_experts", default=0) or 0)
    moe_inter = int(_get(cfg, "moe_intermediate_size", default=1407))
    d.update(num_experts=routed, num_experts_per_tok=int(_get(cfg, "num_experts_per_tok", default=6) or 0),
             moe_intermediate_size=moe_inter, norm_topk_prob=bool(_get(cfg, "norm_topk_prob", default=False)),
             moe_router="softmax_topk", shared_expert_intermediate_size=moe_inter * shared,
             first_moe_layer=int(_get(cfg, "first_k_dense_replace", default=0)),
             moe_layer_freq=int(_get(cfg, "moe_layer_freq", default=1)))
    return {"routed_scaling_factor": float(_get(cfg, "routed_scaling_factor", default=1.0)),
            "topk_method": _get(cfg, "topk_method", default="greedy"),
            "n_group": int(_get(cfg, "n_group", default=1) or 1),
            "topk_group": int(_get(cfg, "topk_group", default=1) or 1), "moe_layer_phase": 0}


def _deepseek(cfg, mt):
    """DeepSeek-MoE (first generation): Llama attention, dense first layers, then routed + shared experts
    (reference: ``python/mlc_llm/model/deepseek/deepseek_model.py:171-208,248-254``)."""
    d = _llama(cfg, mt)
    d["extra"] = _deepseek_moe_fields(cfg, d)
    return d


def _deepseek_v2(cfg, mt):
    """DeepSeek-V2: multi-head latent attention (queries and keys are a no-position part plus a rotary
    part shared by all heads; keys / values are expanded from a low-rank latent) and a mixture of
    experts with shared experts and group-limited routing (reference:
    ``python/mlc_llm/model/deepseek_v2/deepseek_v2_model.py``).  Here every head's q / k is laid out as
    [rotary | no-position] and values are padded to that width, so the paged attention kernels see a
    plain multi-head problem; the latent is expanded before it is cached, or, with ``mla_cache = "latent"``,
    cached itself and attended to through absorbed up-projections (``DecoderModel._attention_mla_latent``)."""
    d = _common(cfg, mt)
    nope = int(_get(cfg, "qk_nope_head_dim", default=128))
    rope = int(_get(cfg, "qk_rope_head_dim", default=64))
    d["head_dim"] = nope + rope
    d["num_key_value_heads"] = d["num_attention_heads"]
    d["partial_rotary_factor"] = rope / (nope + rope)
    scaling = d.get("rope_scaling")
    kind = scaling.get("rope_type", scaling.get("type", "default")) if isinstance(scaling, dict) else "default"
    if kind not in ("default", "linear", "yarn"):
        raise ValueError(f"DeepSeek-V2 rotary scaling {kind!r} is not supported")
    extra = _deepseek_moe_fields(cfg, d)
    if kind == "yarn" and scaling.get("mscale_all_dim"):
        factor = float(scaling["factor"])
        extra["softmax_mscale"] = 1.0 if factor <= 1 else 0.1 * float(scaling["mscale_all_dim"]) * math.log(factor) + 1.0
    extra["mla"] = {"q_lora_rank": _get(cfg, "q_lora_rank"), "kv_lora_rank": int(_get(cfg, "kv_lora_rank", default=512)),
                    "qk_nope_head_dim": nope, "qk_rope_head_dim": rope,
                    "v_head_dim": int(_get(cfg, "v_head_dim", default=128)),
                    # "expanded": per-head keys / values are cached; "latent": the latent itself is cached
                    "cache": str(_get(cfg, "mla_cache", default="expanded"))}
    d["extra"] = extra
    return d


def _nemotron(cfg, mt):
    d = _common(cfg, mt)
    d.update(norm_type="layernorm", norm_weight_offset=1.0, hidden_act="relu2", gated_mlp=False,
             partial_rotary_factor=float(_get(cfg, "partial_rotary_factor", "rope_percent", default=0.5)))
    return d


def _cohere(cfg, mt):
    d = _common(cfg, mt)
    d.update(norm_type="layernorm", parallel_residual=True, shared_input_norm=True,
             tie_word_embeddings=True)
    d["extra"] = {"logit_scale": float(_get(cfg, "logit_scale", default=0.0625)), "norm_no_bias": True}
    return d


def _eagle(cfg, mt):
    """EAGLE draft head: Llama blocks fed with ``fc([embedding ; target feature])``; no final norm and no
    LM head of its own (reference: ``python/mlc_llm/model/eagle/eagle_model.py``)."""
    d = _llama(cfg, mt)
    d["tie_word_embeddings"] = True  # no lm_head parameter: logits come from the target model's head
    d.setdefault("extra", {})
    d["extra"] = dict(d["extra"], eagle=True, eagle_fc_bias=bool(_get(cfg, "bias", default=True)))
    return d


def _medusa(cfg, mt):
    """Medusa heads: ``medusa_num_heads`` stacks of ``medusa_num_layers`` residual SiLU blocks and a
    vocabulary projection, all reading the target's last hidden state (reference:
    ``python/mlc_llm/model/medusa/medusa_model.py``).  There are no decoder layers and no KV cache."""
    h = int(_get(cfg, "hidden_size"))
    return dict(model_type=mt, hidden_size=h, intermediate_size=h, num_hidden_layers=0,
                num_attention_heads=1, num_key_value_heads=1, head_dim=64,
                vocab_size=int(_get(cfg, "vocab_size")), context_window_size=1 << 20,
                prefill_chunk_size=int(_get(cfg, "prefill_chunk_size", default=-1) or -1),
                tie_word_embeddings=True,
                extra={"medusa": {"num_heads": int(_get(cfg, "medusa_num_heads")),
                                  "num_layers": int(_get(cfg, "medusa_num_layers", default=1))}})


def _llava(cfg, mt):
    """LLaVA: a Llama / Mistral language model plus a CLIP vision tower whose projected patch features
    replace the image placeholder in the prompt (reference: ``python/mlc_llm/model/llava/llava_model.py``)."""
    text = dict(cfg.get("text_config") or {})
    text_type = text.get("model_type", "llama")
    if text_type not in ("llama", "mistral"):
        raise ValueError(f"LLaVA with a {text_type!r} language model is not supported")
    for k in ("context_window_size", "prefill_chunk_size", "sliding_window_size", "attention_sink_size",
              "tensor_parallel_shards", "pipeline_parallel_stages", "max_batch_size"):
        if k in cfg and k not in text:
            text[k] = cfg[k]
    text.setdefault("vocab_size", cfg.get("vocab_size", 32064))
    d = _PARSERS[text_type](text, text_type)
    d["model_type"] = mt
    vision = dict(cfg.get("vision_config") or {})
    vision.setdefault("hidden_size", 1024)
    vision.setdefault("intermediate_size", 4096)
    vision.setdefault("num_hidden_layers", 24)
    vision.setdefault("num_attention_heads", 16)
    vision.setdefault("image_size", 336)
    vision.setdefault("patch_size", 14)
    vision.setdefault("hidden_act", "quick_gelu")
    vision.setdefault("layer_norm_eps", 1e-5)
    extra = dict(d.get("extra") or {})
    extra["vision"] = vision
    extra["vision_feature_layer"] = int(cfg.get("vision_feature_layer", -2))
    extra["vision_feature_select_strategy"] = cfg.get("vision_feature_select_strategy", "default")
    extra["projector_hidden_act"] = cfg.get("projector_hidden_act", "gelu")
    extra["image_token_index"] = int(cfg.get("image_token_index", cfg.get("image_token_id", 32000)))
    d["extra"] = extra
    return d


def _qwen35(cfg, mt):
    """Qwen3.5 hybrid: three of every four layers mix tokens with a gated delta-rule recurrence
    (``linear_attention``: short causal convolution, per-head decay, one [key_dim, value_dim] state per
    head), the fourth with softmax attention whose output is gated by a sigmoid of a second query-sized
    projection; RMS norms store the deviation from one and a quarter of each head is rotated
    (reference: ``python/mlc_llm/model/qwen35/qwen35_model.py``)."""
    if isinstance(cfg.get("text_config"), dict):
        outer, cfg = cfg, dict(cfg["text_config"])
        for k in ("context_window_size", "prefill_chunk_size", "tensor_parallel_shards", "max_batch_size"):
            if k in outer and k not in cfg:
                cfg[k] = outer[k]
    cfg = dict(cfg)
    cfg.setdefault("head_dim", 256)
    rp = cfg.get("rope_parameters") if isinstance(cfg.get("rope_parameters"), dict) else {}
    if cfg.get("partial_rotary_factor") is None:
        cfg["partial_rotary_factor"] = rp.get("partial_rotary_factor", 0.25)
    if cfg.get("rope_theta") is None:
        cfg["rope_theta"] = rp.get("rope_theta", 10000000)
    cfg["rope_parameters"] = None  # the sectioned (multimodal) rotary layout equals the plain one for text
    cfg["rope_scaling"] = None
    d = _common(cfg, mt)
    d["attention_bias"] = bool(_get(cfg, "attention_bias", default=False))
    d["qk_norm"] = True
    d["norm_weight_offset"] = 1.0
    d["partial_rotary_factor"] = float(cfg["partial_rotary_factor"])
    n = int(d["num_hidden_layers"])
    interval = int(_get(cfg, "full_attention_interval", default=4))
    types = _get(cfg, "layer_types") or ["full_attention" if (i + 1) % interval == 0 else "linear_attention"
                                          for i in range(n)]
    d["layer_attn_kinds"] = ["mha" if t == "full_attention" else "linear" for t in types]
    extra = dict(d.get("extra") or {})
    extra["gdn"] = {"key_head_dim": int(_get(cfg, "linear_key_head_dim", default=128)),
                    "value_head_dim": int(_get(cfg, "linear_value_head_dim", default=128)),
                    "num_key_heads": int(_get(cfg, "linear_num_key_heads", default=16)),
                    "num_value_heads": int(_get(cfg, "linear_num_value_heads", default=16)),
                    "conv_kernel": int(_get(cfg, "linear_conv_kernel_dim", default=4))}
    extra["attn_output_gate"] = True
    d["extra"] = extra
    return d


def _qwen2_5_vl(cfg, mt):
    """Qwen2.5-VL language model: Qwen2 blocks whose rotary frequency bands are dealt to a (time, height,
    width) position triple (``mrope_section``). For text the three agree, which is plain rotary embedding
    (reference: ``python/mlc_llm/model/qwen2_5_vl/qwen2_5_vl_model.py``; position triples for prompts with
    vision grids: ``ops/mrope.py``)."""
    outer = cfg
    if isinstance(cfg.get("text_config"), dict):
        cfg = dict(cfg["text_config"])
        for k in ("context_window_size", "prefill_chunk_size", "tensor_parallel_shards", "max_batch_size",
                  "pipeline_parallel_stages", "tie_word_embeddings"):
            if k in outer and k not in cfg:
                cfg[k] = outer[k]
    cfg = dict(cfg)
    rp = cfg.get("rope_parameters") if isinstance(cfg.get("rope_parameters"), dict) else (cfg.get("rope_scaling") or {})
    section = rp.get("mrope_section")
    if cfg.get("rope_theta") is None and "rope_theta" in rp:
        cfg["rope_theta"] = rp["rope_theta"]
    cfg["rope_parameters"] = None
    cfg["rope_scaling"] = None
    d = _qwen2(cfg, mt)
    vis = outer.get("vision_config") or {}
    d["extra"] = {"mrope_section": [int(x) for x in section] if section else None,
                  "vision_tokens": {"vision_start_token_id": int(outer.get("vision_start_token_id", 151652)),
                                    "image_token_id": int(outer.get("image_token_id", 151655)),
                                    "video_token_id": int(outer.get("video_token_id", 151656)),
                                    "spatial_merge_size": int(vis.get("spatial_merge_size", 2)),
                                    "tokens_per_second": float(vis.get("tokens_per_second", 2))}}
    return d


def _phi3v(cfg, mt):
    """Phi-3-vision: the Phi-3 language model plus a CLIP tower read through the high-definition tiling
    and 2x2 patch merge (reference: ``python/mlc_llm/model/phi3v/phi3v_model.py``). The vision geometry
    comes from ``vision_config`` when present, else from the CLIP ViT-L/14-336 defaults the HuggingFace
    config implies through ``img_processor``."""
    d = _phi3(cfg, "phi3")
    d["model_type"] = mt
    vision = dict(cfg.get("vision_config") or {})
    proc = cfg.get("img_processor") or {}
    vision.setdefault("hidden_size", int(proc.get("image_dim_out", 1024)))
    vision.setdefault("intermediate_size", 4 * vision["hidden_size"])
    vision.setdefault("num_hidden_layers", 24)
    vision.setdefault("num_attention_heads", 16)
    vision.setdefault("image_size", 336)
    vision.setdefault("patch_size", 14)
    vision.setdefault("hidden_act", "quick_gelu")
    vision.setdefault("layer_norm_eps", 1e-5)
    vision.setdefault("hd_num", int(cfg.get("hd_num", 4)))
    vision["kind"] = "phi3v"
    extra = dict(d.get("extra") or {})
    extra["vision"] = vision
    extra["vision_feature_layer"] = int((proc.get("layer_idx", -2)))
    d["extra"] = extra
    return d


_PARSERS = {
    "phi3_v": _phi3v, "phi3v": _phi3v, "qwen2_5_vl": _qwen2_5_vl, "qwen2_5_vl_text": _qwen2_5_vl, "qwen3_5": _qwen35, "qwen3_5_text": _qwen35, "qwen35": _qwen35,
    "llama": _llama, "mistral": _mistral, "ministral3": _ministral3, "qwen": _qwen, "qwen2": _qwen2, "qwen3": _qwen3,
    "gemma": _gemma, "gemma2": _gemma, "gemma3": _gemma, "gemma3_text": _gemma,
    "phi3": _phi3, "phi": _phi, "phi-msft": _phi, "gpt_neox": _gpt_neox, "gpt2": _gpt2, "gptj": _gptj,
    "gpt_j": _gptj, "glm": _glm, "chatglm": _glm, "rwkv5": _rwkv5, "rwkv6": _rwkv5,
    "gpt_bigcode": _gpt2, "starcoder2": _starcoder2, "stablelm": _stablelm, "stablelm_epoch": _stablelm,
    "olmo": _olmo, "olmo2": _olmo, "mixtral": _mixtral, "qwen2_moe": _qwen_moe, "qwen3_moe": _qwen_moe,
    "llama4": _llama4, "llama4_text": _llama4, "internlm": _internlm, "internlm2": _llama, "baichuan": _llama, "orion": _orion, "minicpm": _minicpm,
    "deepseek": _deepseek, "nemotron": _nemotron, "cohere": _cohere, "deepseek_v2": _deepseek_v2, "eagle": _eagle, "medusa": _medusa, "llava": _llava,
    "aquila": _llama,
    "yi": _llama, "tinyllama": _llama,
}

SUPPORTED_MODEL_TYPES = sorted(_PARSERS)


def from_dict(model_type: str, cfg: Dict[str, Any]) -> ModelConfig:
    """Build a ``ModelConfig`` from a HuggingFace ``config.json`` dict or from the ``model_config``
    section of ``mlc-chat-config.json`` (both spellings of every field are accepted)."""
    mt = model_type.replace("-", "_") if model_type not in _PARSERS else model_type
    if mt not in _PARSERS:
        raise ValueError(f"Unknown model type {model_type!r}; supported: {SUPPORTED_MODEL_TYPES}")
    fields = _PARSERS[mt](cfg, mt)
    known = {f.name for f in dataclasses.fields(ModelConfig)}
    # explicit structural overrides present in the dict win (round trip of our own asdict())
    for k, v in cfg.items():
        if k in known and k not in ("model_type", "extra") and v is not None and k not in fields:
            fields[k] = v
    return ModelConfig(**{k: v for k, v in fields.items() if k in known})
