"""BERT-style bidirectional encoder for embedding models (reference: ``model/bert/bert_model.py``).

Post-LayerNorm blocks, learned position and token-type embeddings, GELU MLP. Linear layers run on
the tcgen05 GEMM through ``ops.linear``; the (non-causal, unpaged) attention of these short batches
uses ``torch.nn.functional.scaled_dot_product_attention``.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, Iterator, List, Tuple

import torch

from .. import ops


@dataclasses.dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"

    @staticmethod
    def from_dict(d: Dict) -> "BertConfig":
        known = {f.name for f in dataclasses.fields(BertConfig)}
        return BertConfig(**{k: v for k, v in d.items() if k in known})


def hf_names(cfg: BertConfig) -> Iterator[Tuple[str, List[str]]]:
    """(our name, HuggingFace names to concatenate on axis 0)."""
    e = "embeddings."
    yield "embed.word", [e + "word_embeddings.weight"]
    yield "embed.position", [e + "position_embeddings.weight"]
    yield "embed.token_type", [e + "token_type_embeddings.weight"]
    yield "embed.ln.weight", [e + "LayerNorm.weight"]
    yield "embed.ln.bias", [e + "LayerNorm.bias"]
    for i in range(cfg.num_hidden_layers):
        s, d = f"encoder.layer.{i}.", f"layers.{i}."
        for leaf in ("weight", "bias"):
            yield d + f"qkv.{leaf}", [s + f"attention.self.{p}.{leaf}" for p in ("query", "key", "value")]
            yield d + f"attn_out.{leaf}", [s + f"attention.output.dense.{leaf}"]
            yield d + f"attn_ln.{leaf}", [s + f"attention.output.LayerNorm.{leaf}"]
            yield d + f"up.{leaf}", [s + f"intermediate.dense.{leaf}"]
            yield d + f"down.{leaf}", [s + f"output.dense.{leaf}"]
            yield d + f"out_ln.{leaf}", [s + f"output.LayerNorm.{leaf}"]


class BertModel:
    def __init__(self, cfg: BertConfig, tensors: Dict[str, torch.Tensor], device: torch.device,
                 dtype: torch.dtype = torch.float16):
        self.cfg, self.device = cfg, device
        self.dtype = dtype if device.type == "cuda" else torch.float32
        self.t = {k: v.to(self.dtype).to(device) for k, v in tensors.items()}
        self.lin = {}
        for i in range(cfg.num_hidden_layers):
            for name in ("qkv", "attn_out", "up", "down"):
                w = self.t[f"layers.{i}.{name}.weight"]
                self.lin[f"layers.{i}.{name}"] = ops.LinearWeight(
                    "dense", w, None, self.t[f"layers.{i}.{name}.bias"], None, w.shape[0], w.shape[1])

    @staticmethod
    def from_hf(path: str, device: torch.device, dtype: torch.dtype = torch.float16) -> "BertModel":
        import json  # pylint: disable=import-outside-toplevel
        import os  # pylint: disable=import-outside-toplevel

        from ..loader.huggingface_loader import HFCheckpoint  # pylint: disable=import-outside-toplevel

        with open(os.path.join(path, "config.json"), encoding="utf-8") as f:
            cfg = BertConfig.from_dict(json.load(f))
        ckpt = HFCheckpoint(path)

        def get(name):
            for pre in ("", "bert."):
                if ckpt.resolve(pre + name) is not None:
                    return ckpt.get(pre + name)
            raise KeyError(name)

        tensors = {dst: torch.cat([get(s) for s in srcs], 0) for dst, srcs in hf_names(cfg)}
        return BertModel(cfg, tensors, device, dtype)

    def _ln(self, x, name, delta=None):
        """LayerNorm of ``x`` (of ``x + delta`` when given): the LayerNorm kernel on the GPU."""
        w, b = self.t[name + ".weight"], self.t[name + ".bias"]
        if delta is None:
            return ops.layernorm(x, w, b, self.cfg.layer_norm_eps)
        shape = x.shape
        res = x.reshape(-1, shape[-1]).contiguous()
        out = ops.layernorm(delta.reshape(-1, shape[-1]).contiguous(), w, b, self.cfg.layer_norm_eps, residual=res)
        return out.reshape(shape)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
        """``input_ids / attention_mask [B, S]`` (mask 1 = token) -> hidden states ``[B, S, H]``."""
        c = self.cfg
        b, s = input_ids.shape
        pos = torch.arange(s, device=input_ids.device)
        x = self.t["embed.word"][input_ids] + self.t["embed.position"][pos][None] + self.t["embed.token_type"][0]
        x = self._ln(x, "embed.ln")
        heads, d = c.num_attention_heads, c.hidden_size // c.num_attention_heads
        bias = (1.0 - attention_mask[:, None, None, :].to(torch.float32)) * -1e4
        # right-padded batches (what the tokenizer produces) are described by their lengths alone
        lens = attention_mask.sum(dim=1).to(torch.int32)
        right_padded = bool((attention_mask.cumsum(1) == torch.arange(1, s + 1, device=attention_mask.device)
                             ).to(attention_mask.dtype).eq(attention_mask).all())
        use_kernel = x.is_cuda and right_padded and x.dtype in (torch.float16, torch.bfloat16)
        for i in range(c.num_hidden_layers):
            p = f"layers.{i}."
            qkv = ops.linear(x.reshape(b * s, -1), self.lin[p + "qkv"]).view(b, s, 3, heads, d)
            if use_kernel:
                a = ops.encoder_attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], key_lens=lens)
                a = a.reshape(b * s, heads * d)
            else:
                q, k, v = (qkv[:, :, j].transpose(1, 2) for j in range(3))
                a = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=bias)
                a = a.transpose(1, 2).reshape(b * s, heads * d).to(x.dtype)
            x = self._ln(x, p + "attn_ln", delta=ops.linear(a, self.lin[p + "attn_out"]).view(b, s, -1))
            h = ops.linear(x.reshape(b * s, -1), self.lin[p + "up"])
            h = ops.activation(h, "gelu" if c.hidden_act == "gelu" else "gelu_tanh")
            x = self._ln(x, p + "out_ln", delta=ops.linear(h, self.lin[p + "down"]).view(b, s, -1))
        return x
