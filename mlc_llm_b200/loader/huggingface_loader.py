"""Read HuggingFace checkpoints (safetensors or torch ``.bin`` shards) and rename / fuse their
tensors into this framework's parameter set.

Reference: ``python/mlc_llm/loader/huggingface_loader.py:26-228`` (lazy shard loading ordered for
file locality, quantise while loading) and ``loader/standard_loader.py:23-152`` (q/k/v concatenated
on axis 0 into ``qkv_proj``; gate/up concatenated into ``gate_up_proj``) plus the per-model
``*_loader.py`` files.  Here one table per naming family produces, for every destination tensor, the
source names and the function that combines them.
"""

from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterator, List, Optional, Tuple

import torch

from ..models.config import ModelConfig
from ..models.transformer import param_specs

Combine = Callable[[List[torch.Tensor]], torch.Tensor]


def _cat0(ts: List[torch.Tensor]) -> torch.Tensor:
    return torch.cat(ts, dim=0)


def _first(ts: List[torch.Tensor]) -> torch.Tensor:
    return ts[0]


def _t(ts: List[torch.Tensor]) -> torch.Tensor:
    return ts[0].t().contiguous()


class Mapping:
    """destination name -> (source names, combine)."""

    def __init__(self) -> None:
        self.items: Dict[str, Tuple[List[str], Combine]] = {}

    def add(self, dst: str, srcs: List[str], fn: Combine = _first) -> None:
        self.items[dst] = (srcs, fn)


# ------------------------------------------------------------------------------------ family tables
def _llama_like(cfg: ModelConfig, m: Mapping, *, prefix: str = "model.", attn: str = "self_attn",
                q="q_proj", k="k_proj", v="v_proj", o="o_proj", mlp="mlp", gate="gate_proj", up="up_proj",
                down="down_proj", in_norm="input_layernorm", post_norm="post_attention_layernorm",
                final_norm="norm", embed="embed_tokens", head="lm_head") -> None:
    specs = param_specs(cfg)

    def has(name: str) -> bool:
        return name in specs

    m.add("model.embed_tokens.weight", [f"{prefix}{embed}.weight"])
    for i in range(cfg.num_hidden_layers):
        s, d = f"{prefix}layers.{i}.", f"model.layers.{i}."
        for suffix in ("weight", "bias"):
            if has(d + f"self_attn.qkv_proj.{suffix}"):
                m.add(d + f"self_attn.qkv_proj.{suffix}",
                      [f"{s}{attn}.{q}.{suffix}", f"{s}{attn}.{k}.{suffix}", f"{s}{attn}.{v}.{suffix}"], _cat0)
            if has(d + f"self_attn.o_proj.{suffix}"):
                m.add(d + f"self_attn.o_proj.{suffix}", [f"{s}{attn}.{o}.{suffix}"])
            if has(d + f"input_layernorm.{suffix}"):
                m.add(d + f"input_layernorm.{suffix}", [f"{s}{in_norm}.{suffix}"])
            if has(d + f"post_attention_layernorm.{suffix}"):
                m.add(d + f"post_attention_layernorm.{suffix}", [f"{s}{post_norm}.{suffix}"])
            if has(d + f"pre_feedforward_layernorm.{suffix}"):
                m.add(d + f"pre_feedforward_layernorm.{suffix}", [f"{s}pre_feedforward_layernorm.{suffix}"])
            if has(d + f"post_feedforward_layernorm.{suffix}"):
                m.add(d + f"post_feedforward_layernorm.{suffix}", [f"{s}post_feedforward_layernorm.{suffix}"])
            if has(d + f"mlp.gate_up_proj.{suffix}"):
                m.add(d + f"mlp.gate_up_proj.{suffix}", [f"{s}{mlp}.{gate}.{suffix}", f"{s}{mlp}.{up}.{suffix}"], _cat0)
            if has(d + f"mlp.up_proj.{suffix}"):
                m.add(d + f"mlp.up_proj.{suffix}", [f"{s}{mlp}.{up}.{suffix}"])
            if has(d + f"mlp.down_proj.{suffix}"):
                m.add(d + f"mlp.down_proj.{suffix}", [f"{s}{mlp}.{down}.{suffix}"])
        if cfg.qk_norm:
            m.add(d + "self_attn.q_norm.weight", [f"{s}{attn}.q_norm.weight"])
            m.add(d + "self_attn.k_norm.weight", [f"{s}{attn}.k_norm.weight"])
    for suffix in ("weight", "bias"):
        if has(f"model.norm.{suffix}"):
            m.add(f"model.norm.{suffix}", [f"{prefix}{final_norm}.{suffix}"])
    if has("lm_head.weight"):
        m.add("lm_head.weight", [f"{head}.weight"])
    if has("lm_head.bias"):
        m.add("lm_head.bias", [f"{head}.bias"])


def _moe_layers(cfg: ModelConfig, m: Mapping, style: str) -> None:
    """Stack per-expert HF matrices into ``e1_e3`` [E, 2I, H] (gate rows then up rows) and ``e2``
    [E, H, I] (reference: ``model/mixtral/mixtral_loader.py``, ``qwen2_moe_loader.py``)."""
    e = cfg.num_experts

    def stack13(ts: List[torch.Tensor]) -> torch.Tensor:
        return torch.stack([torch.cat([ts[2 * j], ts[2 * j + 1]], dim=0) for j in range(e)], dim=0)

    def stack(ts: List[torch.Tensor]) -> torch.Tensor:
        return torch.stack(ts, dim=0)

    for i in range(cfg.num_hidden_layers):
        if not cfg.is_moe_layer(i):
            continue
        d = f"model.layers.{i}.moe."
        if style == "mixtral":
            s = f"model.layers.{i}.block_sparse_moe."
            g, u, dn = "w1", "w3", "w2"
            m.add(d + "gate.weight", [s + "gate.weight"])
        else:
            s = f"model.layers.{i}.mlp."
            g, u, dn = "gate_proj", "up_proj", "down_proj"
            m.add(d + "gate.weight", [s + "gate.weight"])
        srcs13 = []
        for j in range(e):
            srcs13 += [f"{s}experts.{j}.{g}.weight", f"{s}experts.{j}.{u}.weight"]
        m.add(d + "e1_e3.weight", srcs13, stack13)
        m.add(d + "e2.weight", [f"{s}experts.{j}.{dn}.weight" for j in range(e)], stack)
        if cfg.shared_expert_intermediate_size > 0:
            se = "shared_experts" if style == "deepseek" else "shared_expert"
            m.add(d + "shared_expert.gate_up_proj.weight",
                  [s + se + ".gate_proj.weight", s + se + ".up_proj.weight"], _cat0)
            m.add(d + "shared_expert.down_proj.weight", [s + se + ".down_proj.weight"])
            if cfg.shared_expert_gate:
                m.add(d + "shared_expert_gate.weight", [s + "shared_expert_gate.weight"])


def _phi3(cfg: ModelConfig, m: Mapping) -> None:
    _llama_like(cfg, m)
    for i in range(cfg.num_hidden_layers):
        m.add(f"model.layers.{i}.self_attn.qkv_proj.weight", [f"model.layers.{i}.self_attn.qkv_proj.weight"])
        m.add(f"model.layers.{i}.mlp.gate_up_proj.weight", [f"model.layers.{i}.mlp.gate_up_proj.weight"])


def _gpt2(cfg: ModelConfig, m: Mapping) -> None:
    """GPT-2 stores Conv1D weights as [in, out]; they are transposed here (reference:
    ``model/gpt2/gpt2_loader.py``)."""
    pre = "transformer." if cfg.extra.get("hf_prefix", True) else ""
    m.add("model.embed_tokens.weight", [pre + "wte.weight"])
    m.add("model.embed_positions.weight", [pre + "wpe.weight"])
    conv1d = cfg.model_type == "gpt2"
    tw = _t if conv1d else _first
    for i in range(cfg.num_hidden_layers):
        s, d = f"{pre}h.{i}.", f"model.layers.{i}."
        m.add(d + "input_layernorm.weight", [s + "ln_1.weight"])
        m.add(d + "input_layernorm.bias", [s + "ln_1.bias"])
        m.add(d + "self_attn.qkv_proj.weight", [s + "attn.c_attn.weight"], tw)
        m.add(d + "self_attn.qkv_proj.bias", [s + "attn.c_attn.bias"])
        m.add(d + "self_attn.o_proj.weight", [s + "attn.c_proj.weight"], tw)
        m.add(d + "self_attn.o_proj.bias", [s + "attn.c_proj.bias"])
        m.add(d + "post_attention_layernorm.weight", [s + "ln_2.weight"])
        m.add(d + "post_attention_layernorm.bias", [s + "ln_2.bias"])
        m.add(d + "mlp.up_proj.weight", [s + "mlp.c_fc.weight"], tw)
        m.add(d + "mlp.up_proj.bias", [s + "mlp.c_fc.bias"])
        m.add(d + "mlp.down_proj.weight", [s + "mlp.c_proj.weight"], tw)
        m.add(d + "mlp.down_proj.bias", [s + "mlp.c_proj.bias"])
    m.add("model.norm.weight", [pre + "ln_f.weight"])
    m.add("model.norm.bias", [pre + "ln_f.bias"])


def _gptj(cfg: ModelConfig, m: Mapping) -> None:
    """GPT-J rotates interleaved pairs (2i, 2i + 1); the kernels rotate (i, i + rotary_dim / 2).  Attention
    scores do not change when q and k are permuted the same way, so the rows of ``q_proj`` / ``k_proj``
    are reordered per head to [even rotary dims, odd rotary dims, the rest]."""
    hq, d, rot = cfg.num_attention_heads, cfg.head_dim, cfg.rotary_dim
    idx = torch.tensor(list(range(0, rot, 2)) + list(range(1, rot, 2)) + list(range(rot, d)))

    def qkv(ts):
        q, k, v = ts
        perm = lambda w: w.view(hq, d, -1).index_select(1, idx).reshape(hq * d, -1)
        return torch.cat([perm(q), perm(k), v], 0)

    m.add("model.embed_tokens.weight", ["transformer.wte.weight"])
    for i in range(cfg.num_hidden_layers):
        s, dd = f"transformer.h.{i}.", f"model.layers.{i}."
        m.add(dd + "input_layernorm.weight", [s + "ln_1.weight"])
        m.add(dd + "input_layernorm.bias", [s + "ln_1.bias"])
        m.add(dd + "self_attn.qkv_proj.weight",
              [s + "attn.q_proj.weight", s + "attn.k_proj.weight", s + "attn.v_proj.weight"], qkv)
        m.add(dd + "self_attn.o_proj.weight", [s + "attn.out_proj.weight"])
        for suffix in ("weight", "bias"):
            m.add(dd + f"mlp.up_proj.{suffix}", [s + f"mlp.fc_in.{suffix}"])
            m.add(dd + f"mlp.down_proj.{suffix}", [s + f"mlp.fc_out.{suffix}"])
    m.add("model.norm.weight", ["transformer.ln_f.weight"])
    m.add("model.norm.bias", ["transformer.ln_f.bias"])
    m.add("lm_head.weight", ["lm_head.weight"])
    m.add("lm_head.bias", ["lm_head.bias"])


def _deepseek_v2(cfg: ModelConfig, m: Mapping) -> None:
    """Multi-head latent attention tensors.  The checkpoint rotates interleaved pairs of the rotary part
    and puts it last in every head; the kernels rotate half-split pairs of the first ``rotary_dim``
    dimensions, so the rotary rows are de-interleaved and moved to the front of every q head, and
    de-interleaved in place in ``kv_a_proj_with_mqa`` (a permutation shared by q and k leaves the scores
    unchanged)."""
    mla = cfg.extra["mla"]
    hq, nope, rope, rank = cfg.num_attention_heads, mla["qk_nope_head_dim"], mla["qk_rope_head_dim"], mla["kv_lora_rank"]
    deint = list(range(0, rope, 2)) + list(range(1, rope, 2))
    q_idx = torch.tensor([nope + j for j in deint] + list(range(nope)))
    kv_idx = torch.tensor(list(range(rank)) + [rank + j for j in deint])

    def q_rows(ts):
        w = ts[0]
        return w.view(hq, nope + rope, -1).index_select(1, q_idx).reshape(hq * (nope + rope), -1)

    _llama_like(cfg, m)
    for i in range(cfg.num_hidden_layers):
        s = d = f"model.layers.{i}.self_attn."
        if mla.get("q_lora_rank"):
            m.add(d + "q_a_proj.weight", [s + "q_a_proj.weight"])
            m.add(d + "q_a_layernorm.weight", [s + "q_a_layernorm.weight"])
            m.add(d + "q_b_proj.weight", [s + "q_b_proj.weight"], q_rows)
        else:
            m.add(d + "q_proj.weight", [s + "q_proj.weight"], q_rows)
        m.add(d + "kv_a_proj_with_mqa.weight", [s + "kv_a_proj_with_mqa.weight"],
              lambda ts: ts[0].index_select(0, kv_idx))
        m.add(d + "kv_a_layernorm.weight", [s + "kv_a_layernorm.weight"])
        m.add(d + "kv_b_proj.weight", [s + "kv_b_proj.weight"])
        m.add(d + "o_proj.weight", [s + "o_proj.weight"])
    _moe_layers(cfg, m, "deepseek")


def _deinterleave_rows(cfg: ModelConfig, heads: int):
    """Row permutation of a [heads * d, ...] projection that turns interleaved rotary pairs (2i, 2i + 1)
    of the first ``rotary_dim`` dimensions of every head into half-split pairs (i, i + rotary_dim / 2)."""
    d, rot = cfg.head_dim, cfg.rotary_dim
    idx = torch.tensor(list(range(0, rot, 2)) + list(range(1, rot, 2)) + list(range(rot, d)))

    def perm(w: torch.Tensor) -> torch.Tensor:
        return w.reshape(heads, d, -1).index_select(1, idx).reshape(w.shape)

    return perm


def _glm(cfg: ModelConfig, m: Mapping) -> None:
    """HuggingFace ``glm``: Llama names with a fused ``gate_up_proj``; rotary rows de-interleaved."""
    pq, pk = _deinterleave_rows(cfg, cfg.num_attention_heads), _deinterleave_rows(cfg, cfg.num_key_value_heads)
    _llama_like(cfg, m)
    for i in range(cfg.num_hidden_layers):
        s = d = f"model.layers.{i}."
        for suffix in ("weight", "bias"):
            m.add(d + f"self_attn.qkv_proj.{suffix}",
                  [s + f"self_attn.q_proj.{suffix}", s + f"self_attn.k_proj.{suffix}", s + f"self_attn.v_proj.{suffix}"],
                  lambda ts: torch.cat([pq(ts[0]), pk(ts[1]), ts[2]], 0))
        m.add(d + "mlp.gate_up_proj.weight", [s + "mlp.gate_up_proj.weight"])


def _chatglm(cfg: ModelConfig, m: Mapping) -> None:
    """ChatGLM3 checkpoints: ``query_key_value`` is [q; k; v] and ``dense_h_to_4h`` is [gate; up]
    (reference: ``python/mlc_llm/model/chatglm3/chatglm3_loader.py``)."""
    hq, hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    pq, pk = _deinterleave_rows(cfg, hq), _deinterleave_rows(cfg, hkv)

    def qkv(ts):
        w = ts[0]
        q, k, v = w[: hq * hd], w[hq * hd: (hq + hkv) * hd], w[(hq + hkv) * hd:]
        return torch.cat([pq(q), pk(k), v], 0)

    pre = "transformer.encoder."
    m.add("model.embed_tokens.weight", ["transformer.embedding.word_embeddings.weight"])
    for i in range(cfg.num_hidden_layers):
        s, d = f"{pre}layers.{i}.", f"model.layers.{i}."
        m.add(d + "input_layernorm.weight", [s + "input_layernorm.weight"])
        m.add(d + "post_attention_layernorm.weight", [s + "post_attention_layernorm.weight"])
        m.add(d + "self_attn.qkv_proj.weight", [s + "self_attention.query_key_value.weight"], qkv)
        if cfg.attention_bias:
            m.add(d + "self_attn.qkv_proj.bias", [s + "self_attention.query_key_value.bias"], qkv)
        m.add(d + "self_attn.o_proj.weight", [s + "self_attention.dense.weight"])
        m.add(d + "mlp.gate_up_proj.weight", [s + "mlp.dense_h_to_4h.weight"])
        m.add(d + "mlp.down_proj.weight", [s + "mlp.dense_4h_to_h.weight"])
    m.add("model.norm.weight", [pre + "final_layernorm.weight"])
    m.add("lm_head.weight", ["transformer.output_layer.weight"])


def _llama4(cfg: ModelConfig, m: Mapping) -> None:
    """Llama-4: ``feed_forward`` instead of ``mlp``; experts stored as [E, hidden, 2 * inter] / [E, inter, hidden]
    (input-major), transposed here to the [E, out, in] form of the grouped GEMM; interleaved rotary rows
    de-interleaved (reference: ``model/llama4/llama4_loader.py``)."""
    pq, pk = _deinterleave_rows(cfg, cfg.num_attention_heads), _deinterleave_rows(cfg, cfg.num_key_value_heads)
    _llama_like(cfg, m, mlp="feed_forward")
    for i in range(cfg.num_hidden_layers):
        s, d = f"model.layers.{i}.", f"model.layers.{i}."
        m.add(d + "self_attn.qkv_proj.weight",
              [s + "self_attn.q_proj.weight", s + "self_attn.k_proj.weight", s + "self_attn.v_proj.weight"],
              lambda ts: torch.cat([pq(ts[0]), pk(ts[1]), ts[2]], 0))
        if cfg.is_moe_layer(i):
            f = s + "feed_forward."
            m.add(d + "moe.gate.weight", [f + "router.weight"])
            m.add(d + "moe.e1_e3.weight", [f + "experts.gate_up_proj"], lambda ts: ts[0].transpose(1, 2).contiguous())
            m.add(d + "moe.e2.weight", [f + "experts.down_proj"], lambda ts: ts[0].transpose(1, 2).contiguous())
            m.add(d + "moe.shared_expert.gate_up_proj.weight",
                  [f + "shared_expert.gate_proj.weight", f + "shared_expert.up_proj.weight"], _cat0)
            m.add(d + "moe.shared_expert.down_proj.weight", [f + "shared_expert.down_proj.weight"])


def _qwen(cfg: ModelConfig, m: Mapping) -> None:
    """First-generation Qwen: GPT-2 style names, fused ``c_attn``; the MLP computes
    ``c_proj(w1(x) * silu(w2(x)))``, so ``w2`` is the gate (reference: ``model/qwen/qwen_loader.py``)."""
    m.add("model.embed_tokens.weight", ["transformer.wte.weight"])
    for i in range(cfg.num_hidden_layers):
        s, d = f"transformer.h.{i}.", f"model.layers.{i}."
        m.add(d + "input_layernorm.weight", [s + "ln_1.weight"])
        m.add(d + "post_attention_layernorm.weight", [s + "ln_2.weight"])
        m.add(d + "self_attn.qkv_proj.weight", [s + "attn.c_attn.weight"])
        m.add(d + "self_attn.qkv_proj.bias", [s + "attn.c_attn.bias"])
        m.add(d + "self_attn.o_proj.weight", [s + "attn.c_proj.weight"])
        m.add(d + "mlp.gate_up_proj.weight", [s + "mlp.w2.weight", s + "mlp.w1.weight"], _cat0)
        m.add(d + "mlp.down_proj.weight", [s + "mlp.c_proj.weight"])
    m.add("model.norm.weight", ["transformer.ln_f.weight"])
    m.add("lm_head.weight", ["lm_head.weight"])


def _rwkv5(cfg: ModelConfig, m: Mapping) -> None:
    """RWKV-5 / RWKV-6 checkpoints: ``rwkv.`` prefix, mixing weights stored as [1, 1, hidden]; RWKV-5's
    ``time_decay`` is stored before the double exponential; with ``rescale_every`` the output projections of
    block i are divided by 2 ** (i // rescale_every), matching the halving of the activations in the forward
    (reference: ``model/rwkv5/rwkv5_loader.py:41-52``, ``model/rwkv6/rwkv6_loader.py:38-55``)."""
    v6 = int(cfg.extra["rwkv"]) == 6
    nh, hs = cfg.hidden_size // cfg.head_dim, cfg.head_dim
    rescale = int(cfg.extra.get("rescale_every", 0))
    for name, (shape, _kind) in param_specs(cfg).items():
        src = "rwkv." + name[len("model."):] if name.startswith("model.") else name
        if name.endswith("time_decay") and not v6:
            m.add(name, [src], lambda ts: torch.exp(-torch.exp(ts[0].float())).reshape(nh, hs))
        elif name.endswith("time_faaaa"):
            m.add(name, [src], lambda ts: ts[0].float().reshape(nh, hs))
        elif "time_mix_" in name or name.endswith("time_decay") or ("time_maa_" in name and len(shape) == 1):
            m.add(name, [src], lambda ts: ts[0].reshape(-1))
        elif rescale > 0 and (name.endswith("feed_forward.value.weight") or name.endswith("attention.output.weight")):
            block = int(name.split(".")[2])
            m.add(name, [src], lambda ts, t=block // rescale: ts[0] / (2 ** t))
        else:
            m.add(name, [src])


def _gpt_neox(cfg: ModelConfig, m: Mapping) -> None:
    """GPT-NeoX interleaves q, k, v per head inside ``query_key_value`` ([heads, 3, d, hidden]); they
    are regrouped into [q; k; v] (reference: ``model/gpt_neox/gpt_neox_loader.py``)."""
    hq, d = cfg.num_attention_heads, cfg.head_dim

    def regroup_w(ts):
        w = ts[0].view(hq, 3, d, -1)
        return torch.cat([w[:, 0].reshape(hq * d, -1), w[:, 1].reshape(hq * d, -1), w[:, 2].reshape(hq * d, -1)], 0)

    def regroup_b(ts):
        b = ts[0].view(hq, 3, d)
        return torch.cat([b[:, 0].reshape(-1), b[:, 1].reshape(-1), b[:, 2].reshape(-1)], 0)

    m.add("model.embed_tokens.weight", ["gpt_neox.embed_in.weight"])
    for i in range(cfg.num_hidden_layers):
        s, dd = f"gpt_neox.layers.{i}.", f"model.layers.{i}."
        for suffix in ("weight", "bias"):
            m.add(dd + f"input_layernorm.{suffix}", [s + f"input_layernorm.{suffix}"])
            m.add(dd + f"post_attention_layernorm.{suffix}", [s + f"post_attention_layernorm.{suffix}"])
            m.add(dd + f"self_attn.o_proj.{suffix}", [s + f"attention.dense.{suffix}"])
            m.add(dd + f"mlp.up_proj.{suffix}", [s + f"mlp.dense_h_to_4h.{suffix}"])
            m.add(dd + f"mlp.down_proj.{suffix}", [s + f"mlp.dense_4h_to_h.{suffix}"])
        m.add(dd + "self_attn.qkv_proj.weight", [s + "attention.query_key_value.weight"], regroup_w)
        m.add(dd + "self_attn.qkv_proj.bias", [s + "attention.query_key_value.bias"], regroup_b)
    m.add("model.norm.weight", ["gpt_neox.final_layer_norm.weight"])
    m.add("model.norm.bias", ["gpt_neox.final_layer_norm.bias"])
    m.add("lm_head.weight", ["embed_out.weight"])


def _phi(cfg: ModelConfig, m: Mapping) -> None:
    _llama_like(cfg, m, mlp="mlp", up="fc1", down="fc2", final_norm="final_layernorm")
    for i in range(cfg.num_hidden_layers):
        for suffix in ("weight", "bias"):
            m.add(f"model.layers.{i}.self_attn.o_proj.{suffix}", [f"model.layers.{i}.self_attn.dense.{suffix}"])


def _internlm2(cfg: ModelConfig, m: Mapping) -> None:
    """InternLM2 packs ``wqkv`` per KV group as [groups, q_per_group + 2, d, hidden] (reference:
    ``model/internlm2/internlm2_loader.py``)."""
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per = hq // hkv

    def regroup(ts):
        w = ts[0].view(hkv, per + 2, d, -1)
        q = w[:, :per].reshape(hq * d, -1)
        k = w[:, per].reshape(hkv * d, -1)
        v = w[:, per + 1].reshape(hkv * d, -1)
        return torch.cat([q, k, v], 0)

    m.add("model.embed_tokens.weight", ["model.tok_embeddings.weight"])
    for i in range(cfg.num_hidden_layers):
        s, dd = f"model.layers.{i}.", f"model.layers.{i}."
        m.add(dd + "input_layernorm.weight", [s + "attention_norm.weight"])
        m.add(dd + "post_attention_layernorm.weight", [s + "ffn_norm.weight"])
        m.add(dd + "self_attn.qkv_proj.weight", [s + "attention.wqkv.weight"], regroup)
        m.add(dd + "self_attn.o_proj.weight", [s + "attention.wo.weight"])
        m.add(dd + "mlp.gate_up_proj.weight", [s + "feed_forward.w1.weight", s + "feed_forward.w3.weight"], _cat0)
        m.add(dd + "mlp.down_proj.weight", [s + "feed_forward.w2.weight"])
    m.add("model.norm.weight", ["model.norm.weight"])
    m.add("lm_head.weight", ["output.weight"])


def _qwen35(cfg: ModelConfig, m: Mapping) -> None:
    """Qwen3.5: ``q_proj`` holds, per head, the query rows followed by the output-gate rows; the four input
    projections of a linear-attention layer are stacked into two matrices and the depthwise convolution
    loses its singleton channel axis (reference: ``python/mlc_llm/model/qwen35/qwen35_loader.py``)."""
    hq, d = cfg.num_attention_heads, cfg.head_dim
    _llama_like(cfg, m)

    def split_q(part: int):
        return lambda w: w.reshape(hq, 2, d, -1)[:, part].reshape(hq * d, -1)

    for i in range(cfg.num_hidden_layers):
        s = dst = f"model.layers.{i}."
        if cfg.layer_attn_kinds[i] == "linear":
            la = s + "linear_attn."
            m.add(dst + "linear_attn.in_proj_qkvz.weight", [la + "in_proj_qkv.weight", la + "in_proj_z.weight"], _cat0)
            m.add(dst + "linear_attn.in_proj_ba.weight", [la + "in_proj_b.weight", la + "in_proj_a.weight"], _cat0)
            m.add(dst + "linear_attn.conv1d.weight", [la + "conv1d.weight"], lambda ts: ts[0].reshape(ts[0].shape[0], -1))
            for n in ("dt_bias", "A_log", "norm.weight", "out_proj.weight"):
                m.add(dst + "linear_attn." + n, [la + n])
        else:
            a = s + "self_attn."
            m.add(dst + "self_attn.qkv_proj.weight", [a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight"],
                  lambda ts: torch.cat([split_q(0)(ts[0]), ts[1], ts[2]], 0))
            m.add(dst + "self_attn.gate_proj.weight", [a + "q_proj.weight"], lambda ts: split_q(1)(ts[0]).contiguous())


def _baichuan(cfg: ModelConfig, m: Mapping) -> None:
    _llama_like(cfg, m)
    for i in range(cfg.num_hidden_layers):
        m.add(f"model.layers.{i}.self_attn.qkv_proj.weight", [f"model.layers.{i}.self_attn.W_pack.weight"])


def build_mapping(cfg: ModelConfig) -> Mapping:
    m = Mapping()
    mt = cfg.model_type
    if mt in ("gpt2", "gpt_bigcode"):
        _gpt2(cfg, m)
    elif mt == "gpt_neox":
        _gpt_neox(cfg, m)
    elif mt in ("gptj", "gpt_j"):
        _gptj(cfg, m)
    elif mt in ("llama4", "llama4_text"):
        _llama4(cfg, m)
    elif mt == "qwen":
        _qwen(cfg, m)
    elif mt in ("rwkv5", "rwkv6"):
        _rwkv5(cfg, m)
    elif mt == "glm":
        _glm(cfg, m)
    elif mt == "chatglm":
        _chatglm(cfg, m)
    elif mt in ("qwen3_5", "qwen3_5_text", "qwen35"):
        _qwen35(cfg, m)
    elif mt in ("phi3", "phi3_v", "phi3v"):
        _phi3(cfg, m)
    elif mt in ("phi", "phi-msft"):
        _phi(cfg, m)
    elif mt == "internlm2":
        _internlm2(cfg, m)
    elif mt == "baichuan":
        _baichuan(cfg, m)
    elif mt == "starcoder2":
        _llama_like(cfg, m, up="c_fc", down="c_proj")
    elif mt == "mixtral":
        _llama_like(cfg, m)
        _moe_layers(cfg, m, "mixtral")
    elif mt in ("qwen2_moe", "qwen3_moe"):
        _llama_like(cfg, m)
        _moe_layers(cfg, m, "qwen")
    elif mt == "deepseek_v2":
        _deepseek_v2(cfg, m)
    elif mt == "deepseek":
        _llama_like(cfg, m)
        _moe_layers(cfg, m, "deepseek")
    elif mt == "eagle":
        # EAGLE checkpoints name their tensors without the "model." prefix; the resolver tries both
        _llama_like(cfg, m)
        m.add("model.fc.weight", ["fc.weight"])
        if cfg.extra.get("eagle_fc_bias", True):
            m.add("model.fc.bias", ["fc.bias"])
    elif mt == "medusa":
        # same names on both sides (reference: model/medusa/medusa_loader.py, standard loader)
        for name in param_specs(cfg):
            m.add(name, [name])
    else:
        _llama_like(cfg, m)
    # drop destinations the architecture does not have (e.g. dense MLP names on MoE layers)
    specs = param_specs(cfg)
    m.items = {k: v for k, v in m.items.items() if k in specs}
    missing = [k for k in specs if k not in m.items]
    if missing:
        raise ValueError(f"no HuggingFace source known for parameters {missing[:5]} of model type {mt}")
    return m


# ------------------------------------------------------------------------------------ tensor source
class HFCheckpoint:
    """Name -> tensor view over the shards of a HuggingFace checkpoint directory; one shard is open
    at a time."""

    def __init__(self, path: str, lora_adapter: Optional[str] = None):
        self.path = path
        self.name_to_file: Dict[str, str] = {}
        self.lora: Dict[str, Tuple[torch.Tensor, torch.Tensor, float]] = {}
        if lora_adapter is not None:
            self.lora = load_lora_adapter(lora_adapter)
        st_index = os.path.join(path, "model.safetensors.index.json")
        pt_index = os.path.join(path, "pytorch_model.bin.index.json")
        if os.path.isfile(st_index):
            self.name_to_file = dict(json.load(open(st_index, encoding="utf-8"))["weight_map"])
        elif os.path.isfile(os.path.join(path, "model.safetensors")):
            from safetensors import safe_open  # pylint: disable=import-outside-toplevel

            with safe_open(os.path.join(path, "model.safetensors"), "pt") as f:
                self.name_to_file = {k: "model.safetensors" for k in f.keys()}
        elif os.path.isfile(pt_index):
            self.name_to_file = dict(json.load(open(pt_index, encoding="utf-8"))["weight_map"])
        elif os.path.isfile(os.path.join(path, "pytorch_model.bin")):
            sd = torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu", weights_only=True)
            self.name_to_file = {k: "pytorch_model.bin" for k in sd}
            self._open_file, self._open = "pytorch_model.bin", sd
        else:
            raise FileNotFoundError(f"no safetensors or torch checkpoint found under {path}")
        if not hasattr(self, "_open_file"):
            self._open_file: Optional[str] = None
            self._open = None
        # AWQ checkpoints: a linear layer arrives as (qweight, qzeros, scales); it is offered under the
        # name of the 16-bit weight it stands for and expanded when read
        self.awq: Dict[str, str] = {}
        for name in list(self.name_to_file):
            if name.endswith(".qweight"):
                base = name[: -len(".qweight")]
                if base + ".qzeros" in self.name_to_file and base + ".scales" in self.name_to_file \
                        and base + ".weight" not in self.name_to_file:
                    self.awq[base + ".weight"] = base
                    self.name_to_file[base + ".weight"] = self.name_to_file[name]

    def _load_file(self, fname: str) -> None:
        if self._open_file == fname:
            return
        full = os.path.join(self.path, fname)
        if fname.endswith(".safetensors"):
            from safetensors.torch import load_file  # pylint: disable=import-outside-toplevel

            self._open = load_file(full)
        else:
            self._open = torch.load(full, map_location="cpu", weights_only=True)
        self._open_file = fname

    def resolve(self, name: str) -> Optional[str]:
        """Checkpoints differ in whether names carry the ``model.`` / ``transformer.`` prefix."""
        if name in self.name_to_file:
            return name
        for alt in (name.removeprefix("model."), "model." + name, name.removeprefix("transformer."),
                    "transformer." + name, "model.language_model." + name.removeprefix("model."),
                    "language_model." + name, "model.language_model." + name):
            if alt in self.name_to_file:
                return alt
        return None

    def _lora_delta(self, real: str) -> Optional[torch.Tensor]:
        if not self.lora or not real.endswith(".weight"):
            return None
        module = real[: -len(".weight")]
        for cand in (module, module.removeprefix("model."), "model." + module):
            if cand in self.lora:
                a, b, scale = self.lora[cand]
                return (b.float() @ a.float()) * scale
        return None

    def _raw(self, real: str) -> torch.Tensor:
        self._load_file(self.name_to_file[real])
        return self._open[real]

    def get(self, name: str) -> torch.Tensor:
        real = self.resolve(name)
        if real is None:
            raise KeyError(name)
        if real in self.awq:
            from ..quantization import awq_dequantize  # pylint: disable=import-outside-toplevel

            base = self.awq[real]
            w = awq_dequantize(self._raw(base + ".qweight"), self._raw(base + ".qzeros"), self._raw(base + ".scales"))
            delta = self._lora_delta(real)
            return w if delta is None else (w.float() + delta).to(w.dtype)
        delta = self._lora_delta(real)
        if delta is not None:
            self._load_file(self.name_to_file[real])
            w = self._open[real]
            return (w.float() + delta).to(w.dtype)
        self._load_file(self.name_to_file[real])
        return self._open[real]


def load_lora_adapter(adapter_dir: str) -> Dict[str, Tuple[torch.Tensor, torch.Tensor, float]]:
    """Read a PEFT-format LoRA adapter directory (``adapter_config.json`` + ``adapter_model.safetensors``
    or ``adapter_model.bin``): module path -> ``(A [r, in], B [out, r], scale)`` with
    ``scale = lora_alpha / r`` (``/ sqrt(r)`` for rank-stabilised adapters).  Merging is
    ``W += scale * B @ A``, which is what the reference obtains from ``peft``'s ``merge_and_unload``
    (``python/mlc_llm/interface/convert_weight.py:68-98``)."""
    cfg_path = os.path.join(adapter_dir, "adapter_config.json")
    if not os.path.isfile(cfg_path):
        raise ValueError(f"LoRA adapter directory does not exist or has no adapter_config.json: {adapter_dir}")
    acfg = json.load(open(cfg_path, encoding="utf-8"))
    st = os.path.join(adapter_dir, "adapter_model.safetensors")
    if os.path.isfile(st):
        from safetensors.torch import load_file  # pylint: disable=import-outside-toplevel

        sd = load_file(st)
    else:
        sd = torch.load(os.path.join(adapter_dir, "adapter_model.bin"), map_location="cpu", weights_only=True)
    r_default = int(acfg.get("r", 8))
    alpha_default = float(acfg.get("lora_alpha", r_default))
    out: Dict[str, Tuple[torch.Tensor, torch.Tensor, float]] = {}
    for key, a in sd.items():
        if ".lora_A" not in key:
            continue
        module = key.split(".lora_A")[0]
        b_key = key.replace(".lora_A", ".lora_B")
        if b_key not in sd:
            raise ValueError(f"adapter tensor {key} has no lora_B partner")
        short = module.removeprefix("base_model.model.")
        leaf = short.rsplit(".", 1)[-1]
        r = int((acfg.get("rank_pattern") or {}).get(leaf, a.shape[0]))
        alpha = float((acfg.get("alpha_pattern") or {}).get(leaf, alpha_default))
        scale = alpha / (r ** 0.5) if acfg.get("use_rslora") else alpha / r
        w_a, w_b = a, sd[b_key]
        if acfg.get("fan_in_fan_out"):
            w_a, w_b = w_b.t(), w_a.t()
        out[short] = (w_a, w_b, scale)
    if not out:
        raise ValueError(f"no lora_A / lora_B tensors found under {adapter_dir}")
    return out


def iter_mlc_params(path: str, cfg: ModelConfig, lora_adapter: Optional[str] = None
                    ) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield (destination name, full-precision tensor), ordered so that tensors sharing a shard file
    are produced together.  With ``lora_adapter`` the adapter's low-rank updates are merged into the
    tensors they target before any fusing or quantisation."""
    ckpt = HFCheckpoint(path, lora_adapter)
    mapping = build_mapping(cfg)
    tied_head = None

    def file_key(item):
        srcs = item[1][0]
        real = ckpt.resolve(srcs[0])
        return (ckpt.name_to_file.get(real, "~") if real else "~", item[0])

    for dst, (srcs, fn) in sorted(mapping.items.items(), key=file_key):
        if dst == "lm_head.weight" and ckpt.resolve(srcs[0]) is None:
            tied_head = dst  # checkpoint ties the head to the embedding without saying so
            continue
        yield dst, fn([ckpt.get(s) for s in srcs])
    if tied_head is not None:
        emb_src = mapping.items["model.embed_tokens.weight"][0][0]
        yield tied_head, ckpt.get(emb_src)
