"""Config-driven decoder-only transformer over the paged KV cache.

One implementation serves every dense and mixture-of-experts family in ``models/config.py``; the
per-family differences (norm type, biases, qk-norm, partial rotary, gated vs plain MLP, parallel
residual, post-norms, soft-capping, sliding layers, MoE routing) are switches of ``ModelConfig``.
All heavy math goes through ``mlc_llm_b200.ops`` (sm_100a kernels on GPU, fp32 PyTorch on CPU).

Reference: the Relax modules of ``python/mlc_llm/model/llama/llama_model.py:106-423`` (layer math,
tensor-parallel sharding, batch_prefill / batch_decode / batch_verify entry points) and
``model/mixtral/mixtral_model.py:64-168`` (MoE block).
"""

from __future__ import annotations

import dataclasses
import os
import math
from typing import Dict, List, Optional

import torch

from .. import ops
from .. import quantization as Q
from ..ops import LinearWeight
from .config import ModelConfig


@dataclasses.dataclass
class BatchInfo:
    """Device-resident index arrays of one forward call (built from the KV manager's plan)."""

    positions: torch.Tensor
    slots: torch.Tensor
    q_seq: torch.Tensor
    q_kvlen: torch.Tensor
    page_indptr: torch.Tensor
    page_indices: torch.Tensor
    q_kvstart: Optional[torch.Tensor] = None
    tree_mask: Optional[torch.Tensor] = None
    attn_plan: object = None  # tensor-core attention schedule (GPU only)
    num_tokens: int = 0


class ParamStore:
    """Named parameters in their run-time form (dense tensors and ``LinearWeight`` objects)."""

    def __init__(self):
        self.tensors: Dict[str, torch.Tensor] = {}
        self.linears: Dict[str, LinearWeight] = {}

    def nbytes(self) -> int:
        total = sum(t.numel() * t.element_size() for t in self.tensors.values())
        for lw in self.linears.values():
            total += lw.w.numel() * lw.w.element_size()
            if lw.scale is not None:
                total += lw.scale.numel() * lw.scale.element_size()
            if lw.bias is not None:
                total += lw.bias.numel() * lw.bias.element_size()
            if getattr(lw, "_tiles", None) is not None:
                total += lw._tiles.numel()  # pylint: disable=protected-access
        return total


class DecoderModel:
    """A (tensor-parallel shard of a) decoder model plus its paged KV cache."""

    def __init__(self, config: ModelConfig, quant: Q.Quantization, params: ParamStore,
                 device: torch.device, comm=None, layer_range: Optional[range] = None):
        self.cfg = config
        self.quant = quant
        self.p = params
        self.device = device
        self.comm = comm  # tensor-parallel communicator (None when world == 1)
        self.tp = getattr(comm, "tp_size", None) or (comm.world_size if comm is not None else 1)
        self.dtype = quant.torch_dtype
        self.hq = config.num_attention_heads // self.tp
        self.hkv = max(1, config.num_key_value_heads // self.tp)
        self.d = config.head_dim
        self.layers = layer_range if layer_range is not None else range(config.num_hidden_layers)
        self.first_stage = self.layers.start == 0
        self.last_stage = self.layers.stop == config.num_hidden_layers
        self.kv_pages: Optional[torch.Tensor] = None
        self.page = 16
        self.sm_scale = (config.query_pre_attn_scalar ** -0.5 if config.query_pre_attn_scalar > 0
                         else self.d ** -0.5)
        self.inv_freq = None
        self.inv_freq_local = None
        self.rope_attn_factor = 1.0
        if config.position_embedding == "rope":
            self.inv_freq = ops.reference.rope_inv_freq(config.rotary_dim, config.rope_theta,
                                                        config.rope_scaling).to(device)
            if config.rope_local_theta > 0:
                self.inv_freq_local = ops.reference.rope_inv_freq(
                    config.rotary_dim, config.rope_local_theta, None).to(device)
            self.rope_attn_factor = ops.reference.rope_attention_factor(config.rope_scaling)
            if config.extra.get("softmax_mscale"):
                # YaRN checkpoints trained with `mscale_all_dim` fold its square into the softmax scale
                self.sm_scale *= float(config.extra["softmax_mscale"]) ** 2

        # Latent attention caches either per-head keys / values expanded from the latent ("expanded") or the
        # latent itself plus the shared rotary key ("latent": one row of rope + rank values per token and layer
        # for all heads, queries and outputs go through the absorbed up-projections).
        mla = config.extra.get("mla")
        self.mla_latent = bool(mla) and (os.environ.get("MLCB_MLA_CACHE") or mla.get("cache", "expanded")) == "latent"
        self._mla_absorbed: dict = {}
        if self.mla_latent:
            self.cache_kv_heads = 1
            self.cache_head_dim = (mla["qk_rope_head_dim"] + mla["kv_lora_rank"] + 1) // 2  # K and V halves of a row

    # ------------------------------------------------------------------ KV cache
    def create_kv_cache(self, num_pages: int, page_size: int = 16) -> None:
        self.page = page_size
        n = len(self.layers)
        if self.mla_latent:
            m = self.cfg.extra["mla"]
            self.kv_pages = torch.zeros(n, num_pages, 1, 1, page_size, m["qk_rope_head_dim"] + m["kv_lora_rank"],
                                        dtype=self.kv_dtype, device=self.device)
            return
        self.kv_pages = torch.zeros(n, num_pages, 2, self.hkv, page_size, self.d, dtype=self.kv_dtype,
                                    device=self.device)

    def _kv_layer(self, li: int) -> int:
        """Index of layer ``li`` in ``kv_pages`` (models that cache only some layers override this)."""
        return li - self.layers.start

    @property
    def kv_dtype(self) -> torch.dtype:
        return self.dtype if self.dtype != torch.float32 or self.device.type == "cpu" else torch.float16

    def kv_bytes_per_token(self) -> int:
        es = 2 if self.kv_dtype != torch.float32 else 4
        if self.mla_latent:
            m = self.cfg.extra["mla"]
            return (m["qk_rope_head_dim"] + m["kv_lora_rank"]) * len(self.layers) * es
        return 2 * self.hkv * self.d * len(self.layers) * es

    def copy_pages(self, pairs: torch.Tensor) -> None:
        """(src, dst) page copies for copy-on-write, applied to every layer."""
        if pairs.numel() == 0:
            return
        if self.kv_pages.is_cuda and pairs.dtype == torch.int32 and pairs.is_cuda:
            # one launch for all layers; destinations are freshly allocated pages, so no pair reads what
            # another writes
            from ..ops._lib import check, lib, ptr, stream_ptr  # pylint: disable=import-outside-toplevel
            import ctypes  # pylint: disable=import-outside-toplevel

            kv = self.kv_pages
            es = kv.element_size()
            check(lib().mlcb_page_copy(ptr(kv), ptr(pairs.contiguous()), ctypes.c_int(pairs.numel() // 2),
                                       ctypes.c_int(kv.shape[0]), ctypes.c_longlong(kv.stride(1) * es),
                                       ctypes.c_longlong(kv.stride(0) * es), stream_ptr()), "mlcb_page_copy")
            return
        src, dst = pairs[0::2].long(), pairs[1::2].long()
        self.kv_pages[:, dst] = self.kv_pages[:, src]

    def move_tokens(self, moves: torch.Tensor) -> None:
        """(src_slot, dst_slot) token moves (tree commit), applied to every layer. A destination may be
        another move's source (accepted nodes slide towards the front), so all rows are gathered before any
        is written: indexing does that, one kernel moving rows in place would not."""
        if moves.numel() == 0:
            return
        src, dst = moves[0::2].long(), moves[1::2].long()
        sp, so = src // self.page, src % self.page
        dp, do = dst // self.page, dst % self.page
        self.kv_pages[:, dp, :, :, do, :] = self.kv_pages[:, sp, :, :, so, :]

    # ------------------------------------------------------------------ pieces
    def _norm(self, x, name, eps=None):
        c = self.cfg
        w = self.p.tensors.get(name + ".weight")
        if c.norm_type == "layernorm":
            b = self.p.tensors.get(name + ".bias")
            if w is None:
                w = torch.ones(x.shape[-1], dtype=x.dtype, device=x.device)
            elif c.norm_weight_offset:
                w = w + c.norm_weight_offset  # "LayerNorm1P": the stored weight is the deviation from one
            return ops.layernorm(x, w, b, c.rms_norm_eps)
        return ops.rmsnorm(x, w, c.rms_norm_eps, c.norm_weight_offset)

    def _add_norm(self, delta, residual, name):
        """residual += delta; returns norm(residual)."""
        c = self.cfg
        if c.norm_type == "rms":
            return ops.add_rmsnorm(delta, residual, self.p.tensors[name + ".weight"], c.rms_norm_eps,
                                   c.norm_weight_offset)
        if c.norm_type == "layernorm" and not c.norm_weight_offset and (name + ".weight") in self.p.tensors \
                and delta.is_contiguous() and residual.is_contiguous():
            return ops.layernorm(delta, self.p.tensors[name + ".weight"], self.p.tensors.get(name + ".bias"),
                                 c.rms_norm_eps, residual=residual)
        residual.add_(delta)
        return self._norm(residual, name)

    def embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        table = self.p.linears.get("model.embed_tokens") or self.p.tensors["model.embed_tokens.weight"]
        x = ops.embed(token_ids, table, c.hidden_size, self.dtype, c.embedding_scale)
        return x  # learned positions are added in forward(), where positions are known

    def _attention_mla(self, li: int, h: torch.Tensor, b: BatchInfo) -> torch.Tensor:
        """Multi-head latent attention with the latent expanded before caching: q / k heads are
        [rotary | no-position] (the rotary key part is shared by all heads), values are zero-padded to
        the q / k width, and the paged kernels run an ordinary multi-head problem. Under tensor parallelism
        a rank holds ``num_heads / tp`` heads of the up-projections and of ``o_proj``'s input; the latent
        projections are computed whole on every rank (they are small) and the caller all-reduces the output."""
        c, m = self.cfg, self.cfg.extra["mla"]
        pre = f"model.layers.{li}.self_attn."
        t = h.shape[0]
        hq, d = self.hq, self.d
        nope, rope, vd, rank = m["qk_nope_head_dim"], m["qk_rope_head_dim"], m["v_head_dim"], m["kv_lora_rank"]
        if m.get("q_lora_rank"):
            qa = ops.linear(h, self.p.linears[pre + "q_a_proj"])
            qa = ops.rmsnorm(qa, self.p.tensors[pre + "q_a_layernorm.weight"], c.rms_norm_eps, 0.0)
            q = ops.linear(qa, self.p.linears[pre + "q_b_proj"])
        else:
            q = ops.linear(h, self.p.linears[pre + "q_proj"])
        ckv = ops.linear(h, self.p.linears[pre + "kv_a_proj_with_mqa"])
        latent = ops.rmsnorm(ckv[:, :rank].contiguous(), self.p.tensors[pre + "kv_a_layernorm.weight"],
                             c.rms_norm_eps, 0.0)
        if self.mla_latent:
            return self._attention_mla_latent(li, q.view(t, hq, d), ckv[:, rank:], latent, b)
        kv = ops.linear(latent, self.p.linears[pre + "kv_b_proj"]).view(t, hq, nope + vd)
        k = torch.cat([ckv[:, rank:].unsqueeze(1).expand(t, hq, rope), kv[..., :nope]], dim=-1)
        v = torch.nn.functional.pad(kv[..., nope:], (0, d - vd))
        qkv = torch.cat([q.view(t, hq, d), k, v], dim=1).reshape(t, 3 * hq * d).contiguous()
        ctx = self._attention_core(li, qkv, b).view(t, hq, d)[..., :vd].reshape(t, hq * vd).contiguous()
        return ops.linear(ctx, self.p.linears[pre + "o_proj"])

    def _mla_up_projections(self, li: int):
        """Per-head key and value up-projections of layer ``li`` as dense batched-matmul operands:
        ``w_uk [hq, nope, rank]`` (absorbed into the queries) and ``w_uv_t [hq, rank, v]`` (applied to the
        attention-weighted latents)."""
        got = self._mla_absorbed.get(li)
        if got is None:
            m = self.cfg.extra["mla"]
            nope, vd, rank = m["qk_nope_head_dim"], m["v_head_dim"], m["kv_lora_rank"]
            lw = self.p.linears[f"model.layers.{li}.self_attn.kv_b_proj"]
            w = lw.dense(self.dtype).view(self.hq, nope + vd, rank)
            got = (w[:, :nope, :].contiguous(), w[:, nope:, :].transpose(1, 2).contiguous())
            if lw.kind != "dense":
                lw._dense = None  # pylint: disable=protected-access  (the two copies above replace it)
            self._mla_absorbed[li] = got
        return got

    def _attention_mla_latent(self, li: int, q: torch.Tensor, k_rope: torch.Tensor, latent: torch.Tensor,
                              b: BatchInfo) -> torch.Tensor:
        """Latent attention over the compressed cache. ``q [T, hq, rope + nope]`` (rotary part first),
        ``k_rope [T, rope]`` (unrotated, shared by all heads), ``latent [T, rank]`` (normalised).
        Scores are ``q_rope . k_rope + (q_nope W_uk) . latent``, the context is ``(softmax . latent) W_uv``:
        the same numbers as expanding keys and values from the latent, without ever storing them."""
        c, m = self.cfg, self.cfg.extra["mla"]
        pre = f"model.layers.{li}.self_attn."
        t, hq = q.shape[0], self.hq
        nope, rope, vd, rank = m["qk_nope_head_dim"], m["qk_rope_head_dim"], m["v_head_dim"], m["kv_lora_rank"]
        w_uk, w_uv_t = self._mla_up_projections(li)
        local = self._kv_layer(li)
        cache = self.kv_pages[local]
        # rotate the rotary parts with the rotary kernel (hq query heads and one key head of width `rope`;
        # slot -1: nothing is appended by that call)
        rot = torch.cat([q[..., :rope].reshape(t, hq * rope), k_rope, torch.zeros_like(k_rope)], dim=1).contiguous()
        if self.inv_freq is not None:
            ops.rope_append(rot, cache, b.positions, torch.full_like(b.slots, -1), self.inv_freq, hq, 1, rope, rope,
                            self.page, self.rope_attn_factor)
        q_lat = torch.bmm(q[..., rope:].transpose(0, 1), w_uk).transpose(0, 1)          # [T, hq, rank]
        q_abs = torch.cat([rot[:, : hq * rope].view(t, hq, rope), q_lat], dim=-1).contiguous()
        rows = torch.cat([rot[:, hq * rope: (hq + 1) * rope], latent], dim=-1).to(cache.dtype).contiguous()
        ops.mla_append(rows, cache, b.slots, self.page)
        ctx = ops.mla_attention(q_abs.to(cache.dtype), cache, b.q_seq, b.q_kvlen, b.page_indptr, b.page_indices,
                                rope, rank, self.page, self.sm_scale, q_kvstart=b.q_kvstart, tree_mask=b.tree_mask)
        v = torch.bmm(ctx.to(self.dtype).transpose(0, 1), w_uv_t).transpose(0, 1)       # [T, hq, v]
        return ops.linear(v.reshape(t, hq * vd).contiguous(), self.p.linears[pre + "o_proj"])

    def _attention(self, li: int, h: torch.Tensor, b: BatchInfo) -> torch.Tensor:
        if self.cfg.extra.get("mla"):
            return self._attention_mla(li, h, b)
        pre = f"model.layers.{li}.self_attn."
        qkv = ops.linear(h, self.p.linears[pre + "qkv_proj"])
        return ops.linear(self._attention_core(li, qkv, b), self.p.linears[pre + "o_proj"])

    def _attention_core(self, li: int, qkv: torch.Tensor, b: BatchInfo) -> torch.Tensor:
        """q/k norms, RoPE + KV append and paged attention on a fused ``qkv`` projection; returns
        the attention context ``[T, hq * d]`` (input of ``o_proj``)."""
        c = self.cfg
        pre = f"model.layers.{li}.self_attn."
        hq, hkv, d = self.hq, self.hkv, self.d
        if c.qk_norm and c.extra.get("qk_norm_full"):
            # OLMo-2 normalises the whole q / k projection, not each head
            if self.tp > 1:
                raise NotImplementedError("full-width q/k norm is not supported with tensor parallelism")
            nq, nk = hq * d, hkv * d
            qkv[:, :nq] = ops.rmsnorm(qkv[:, :nq].contiguous(), self.p.tensors[pre + "q_norm.weight"],
                                      c.rms_norm_eps, c.norm_weight_offset)
            qkv[:, nq:nq + nk] = ops.rmsnorm(qkv[:, nq:nq + nk].contiguous(), self.p.tensors[pre + "k_norm.weight"],
                                             c.rms_norm_eps, c.norm_weight_offset)
        elif c.qk_norm:
            t = qkv.shape[0]
            heads = qkv.view(t, hq + 2 * hkv, d)
            qn = ops.rmsnorm(heads[:, :hq].reshape(-1, d), self.p.tensors[pre + "q_norm.weight"],
                             c.rms_norm_eps, c.norm_weight_offset)
            kn = ops.rmsnorm(heads[:, hq:hq + hkv].reshape(-1, d), self.p.tensors[pre + "k_norm.weight"],
                             c.rms_norm_eps, c.norm_weight_offset)
            heads[:, :hq] = qn.view(t, hq, d)
            heads[:, hq:hq + hkv] = kn.view(t, hkv, d)
        kind = c.layer_attn_kinds[li] if c.layer_attn_kinds is not None else None
        sliding = kind == "mha_sliding"
        inv = self.inv_freq_local if (sliding and self.inv_freq_local is not None) else self.inv_freq
        local = self._kv_layer(li)
        kvstart = b.q_kvstart
        l4 = c.extra.get("llama4")
        if l4 is not None:
            t = qkv.shape[0]
            heads = qkv.view(t, hq + 2 * hkv, d)
            if kind == "mha_nope":
                # position-free layer: no rotation; queries are scaled by a temperature that grows with
                # the position (llama4_model.py: attn_temperature_tuning)
                ops.rope_append(qkv, self.kv_pages[local], b.positions, b.slots, None, hq, hkv, d, 0, self.page)
                if l4["attn_temperature_tuning"]:
                    pos = b.positions.float()
                    scale = torch.log1p(torch.floor((pos + 1.0) / l4["floor_scale"])) * l4["attn_scale"] + 1.0
                    heads[:, :hq] = (heads[:, :hq].float() * scale.view(t, 1, 1)).to(qkv.dtype)
            else:
                if l4["use_qk_norm"]:
                    # rotate without appending, L2-normalise q and k per head (no weight), then append
                    ops.rope_append(qkv, self.kv_pages[local], b.positions, torch.full_like(b.slots, -1), inv,
                                    hq, hkv, d, c.rotary_dim, self.page)
                    qk = heads[:, : hq + hkv].float()
                    qk = qk * torch.rsqrt(qk.pow(2).mean(-1, keepdim=True) + c.rms_norm_eps)
                    heads[:, : hq + hkv] = qk.to(qkv.dtype)
                    ops.rope_append(qkv, self.kv_pages[local], b.positions, b.slots, None, hq, hkv, d, 0, self.page)
                else:
                    ops.rope_append(qkv, self.kv_pages[local], b.positions, b.slots, inv, hq, hkv, d,
                                    c.rotary_dim, self.page)
                chunk = int(l4["attention_chunk_size"])
                if chunk > 0:  # a token attends inside its own chunk of positions only
                    kvstart = (torch.div(b.q_kvlen - 1, chunk, rounding_mode="floor") * chunk).to(torch.int32)
        else:
            ops.rope_append(qkv, self.kv_pages[local], b.positions, b.slots, inv, hq, hkv, d,
                            c.rotary_dim if inv is not None else 0, self.page,
                            1.0 if inv is self.inv_freq_local else self.rope_attn_factor)
            qs = c.extra.get("q_pos_scale")
            if qs:  # queries grow with the logarithm of how many trained windows the position lies beyond
                t = qkv.shape[0]
                scale = 1.0 + qs["beta"] * torch.log1p(torch.floor(b.positions.float() / qs["window"]))
                q = qkv.view(t, hq + 2 * hkv, d)[:, :hq]
                q.copy_((q.float() * scale.view(t, 1, 1)).to(qkv.dtype))
        if sliding:
            w = int(c.extra.get("layer_sliding_window", 4096))
            kvstart = torch.clamp(b.q_kvlen - w, min=0).to(torch.int32)
        out = ops.paged_attention(qkv[:, : hq * d], self.kv_pages[local], b.q_seq, b.q_kvlen, b.page_indptr,
                                  b.page_indices, hq, hkv, d, self.page, self.sm_scale, q_kvstart=kvstart,
                                  sink=max(0, c.attention_sink_size) if kvstart is not None and not sliding
                                  and l4 is None else 0,
                                  tree_mask=b.tree_mask, softcap=c.attn_logit_softcap, plan=b.attn_plan)
        return out.reshape(out.shape[0], hq * d)

    def _mlp(self, li: int, h: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        if c.is_moe_layer(li):
            from .moe import moe_block  # pylint: disable=import-outside-toplevel

            return moe_block(self, li, h)
        pre = f"model.layers.{li}.mlp."
        if c.gated_mlp:
            g = ops.linear(h, self.p.linears[pre + "gate_up_proj"])
            a = ops.act_mul(g, "silu" if c.hidden_act == "silu" else "gelu")
        else:
            u = ops.linear(h, self.p.linears[pre + "up_proj"])
            a = ops.activation(u, c.hidden_act if c.hidden_act in ("relu2", "gelu", "silu") else "gelu_tanh")
        return ops.linear(a, self.p.linears[pre + "down_proj"])

    def _reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.comm is not None and self.tp > 1:
            self.comm.all_reduce(x)
        return x

    # ------------------------------------------------------------------ fused tensor parallelism
    def enable_fused(self, fused) -> bool:
        """Use the fused GEMM+collective kernels (``parallel.fused.FusedCollectives``) when the
        architecture has the plain pre-norm RMSNorm block structure they implement; otherwise the
        model keeps the NCCL all-reduce path. Returns whether the fused path is on."""
        c = self.cfg
        # mixture-of-experts layers qualify when whole experts live on the ranks (their exchange is this
        # package's kernels, the block's output then only has to be added to the residual stream) and no
        # shared expert needs a reduction of its own
        moe_ok = c.num_experts == 0 or (
            getattr(self, "ep", None) is not None and getattr(fused, "mode", "") == "ar"
            and c.shared_expert_intermediate_size <= 0 and c.moe_router != "llama4_sigmoid")
        plain = (c.norm_type == "rms" and not c.parallel_residual and not c.post_attention_norm
                 and not c.post_mlp_norm and not c.extra.get("no_pre_norm") and moe_ok
                 and c.gated_mlp and c.position_embedding != "learned" and "residual_scale" not in c.extra
                 and "mla" not in c.extra and "llama4" not in c.extra
                 and self.dtype in (torch.float16, torch.bfloat16))
        # a pipeline stage hands the whole residual stream to the next one: only the all-reduce form keeps it
        # whole on every rank
        if not (self.first_stage and self.last_stage) and getattr(fused, "mode", "") != "ar":
            plain = False
        self.fused = fused if plain else None
        return self.fused is not None

    def _forward_fused(self, x: torch.Tensor, b: BatchInfo) -> torch.Tensor:
        """Forward with the residual stream scattered over the ranks (each keeps the rows it owns).
        Per layer: qkv (all-gather form) -> attention -> o_proj (reduce-scatter form, + residual +
        post-attention norm) -> gate_up (all-gather form) -> activation -> down_proj (reduce-scatter
        form, + residual + next layer's input norm, or the final norm). Returns the final normalised
        hidden states of all rows."""
        c, f = self.cfg, self.fused
        f.begin(x.shape[0])
        x = x.contiguous()
        f.scatter_residual(x)
        layers = list(self.layers)
        if f.mode == "ar":
            # all-reduce form: every rank keeps the whole residual stream; the row-parallel GEMMs reduce
            # over the ranks in their own tail (+ residual + norm), the column-parallel ones are plain
            h = self._norm(x, f"model.layers.{layers[0]}.input_layernorm")
            for pos, li in enumerate(layers):
                pre = f"model.layers.{li}."
                qkv = ops.linear(h, self.p.linears[pre + "self_attn.qkv_proj"])
                ctx = self._attention_core(li, qkv, b)
                h = f.gemm_ar_norm(ctx, self.p.linears[pre + "self_attn.o_proj"],
                                   self.p.tensors[pre + "post_attention_layernorm.weight"], c.rms_norm_eps,
                                   c.norm_weight_offset)
                if pos + 1 < len(layers):
                    nxt = f"model.layers.{layers[pos + 1]}.input_layernorm"
                elif self.last_stage:
                    nxt = "model.norm"
                else:
                    # the next stage normalises with its own first layer's weight; this call's norm output is
                    # not used, only the residual it leaves behind
                    nxt = pre + "post_attention_layernorm"
                if c.is_moe_layer(li):
                    # expert-parallel block: every rank ends up with the output of all tokens, which joins the
                    # residual stream by the add + norm kernel (no collective of its own)
                    from .moe import moe_block  # pylint: disable=import-outside-toplevel

                    out = moe_block(self, li, h)
                    h = ops.add_rmsnorm(out.contiguous(), f.residual[: x.shape[0]], self.p.tensors[nxt + ".weight"],
                                        c.rms_norm_eps, c.norm_weight_offset)
                    continue
                g = ops.linear(h, self.p.linears[pre + "mlp.gate_up_proj"])
                a = ops.act_mul(g, "silu" if c.hidden_act == "silu" else "gelu")
                h = f.gemm_ar_norm(a, self.p.linears[pre + "mlp.down_proj"], self.p.tensors[nxt + ".weight"],
                                   c.rms_norm_eps, c.norm_weight_offset)
            f.end()
            if not self.last_stage:
                self._final_normed = None
                return f.residual[: x.shape[0]].clone()
            self._final_normed = h
            return h
        h = self._norm(x, f"model.layers.{layers[0]}.input_layernorm")
        for pos, li in enumerate(layers):
            pre = f"model.layers.{li}."
            if pos == 0:
                qkv = ops.linear(h, self.p.linears[pre + "self_attn.qkv_proj"])
            else:
                qkv = f.gemm_ag(self.p.linears[pre + "self_attn.qkv_proj"])
            ctx = self._attention_core(li, qkv, b)
            f.gemm_rs_norm(ctx, self.p.linears[pre + "self_attn.o_proj"],
                           self.p.tensors[pre + "post_attention_layernorm.weight"], c.rms_norm_eps,
                           c.norm_weight_offset)
            g = f.gemm_ag(self.p.linears[pre + "mlp.gate_up_proj"])
            a = ops.act_mul(g, "silu" if c.hidden_act == "silu" else "gelu")
            nxt = f"model.layers.{layers[pos + 1]}.input_layernorm" if pos + 1 < len(layers) else "model.norm"
            f.gemm_rs_norm(a, self.p.linears[pre + "mlp.down_proj"], self.p.tensors[nxt + ".weight"],
                           c.rms_norm_eps, c.norm_weight_offset)
        out = f.wait_gather()
        f.end()
        self._final_normed = out
        return out

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, b: BatchInfo) -> torch.Tensor:
        """``x``: embeddings (first stage) or the previous stage's hidden state, ``[T, H]``.
        Returns the residual stream after this stage's layers (final norm NOT applied)."""
        c = self.cfg
        if getattr(self, "fused", None) is not None and x.is_cuda and x.shape[0] > 0:
            return self._forward_fused(x, b)
        if c.position_embedding == "learned" and self.first_stage:
            x = x + self.p.tensors["model.embed_positions.weight"][b.positions.long()].to(x.dtype)
        x = x.contiguous()
        no_pre_norm = bool(c.extra.get("no_pre_norm"))
        rs = float(c.extra.get("residual_scale", 1.0))  # MiniCPM scales every residual branch
        pending = None  # branch output not yet added to the residual stream
        for li in self.layers:
            pre = f"model.layers.{li}."
            if c.parallel_residual:
                if pending is not None:
                    x = x + pending
                    pending = None
                h1 = self._norm(x, pre + "input_layernorm")
                h2 = h1 if c.shared_input_norm else self._norm(x, pre + "post_attention_layernorm")
                attn = self._attention(li, h1, b)
                mlp = self._mlp(li, h2)
                pending = self._reduce(attn + mlp)
                self._mlp_complete = False
                continue
            # ---- attention block
            if no_pre_norm:
                if pending is not None:
                    x = x + pending
                    pending = None
                h = x
            elif pending is None:
                # the first block of an EAGLE head reads the fused input as it is
                h = x if (c.extra.get("eagle") and li == 0) else self._norm(x, pre + "input_layernorm")
            else:
                h = self._add_norm(pending, x, pre + "input_layernorm")
                pending = None
            attn = self._reduce(self._attention(li, h, b))
            if rs != 1.0:
                attn = attn * rs
            if c.post_attention_norm:
                attn = self._norm(attn, pre + ("post_attention_layernorm" if (c.post_mlp_norm)
                                               else "post_attention_norm"))
            # ---- MLP block
            if no_pre_norm:
                x = x + attn
                h = x
            else:
                mlp_norm = "pre_feedforward_layernorm" if (c.post_attention_norm and not no_pre_norm) \
                    else "post_attention_layernorm"
                h = self._add_norm(attn, x, pre + mlp_norm)
            mlp = self._mlp(li, h)
            if getattr(self, "_mlp_complete", False):
                self._mlp_complete = False
            else:
                mlp = self._reduce(mlp)
            if rs != 1.0:
                mlp = mlp * rs
            if c.post_mlp_norm:
                mlp = self._norm(mlp, pre + "post_feedforward_layernorm")
            pending = mlp
        if pending is not None:
            if self.last_stage and c.norm_type == "rms" and not no_pre_norm and not c.extra.get("eagle"):
                self._final_normed = self._add_norm(pending, x, "model.norm")
                return x
            x = x + pending
        self._final_normed = None
        return x

    # ------------------------------------------------------------------ speculative draft heads
    def final_features(self, hidden: torch.Tensor) -> torch.Tensor:
        """Final-normed hidden states of all rows of the latest forward (the "features" that EAGLE and
        Medusa heads consume); must be called before :meth:`logits` consumes the cached tensor."""
        normed = getattr(self, "_final_normed", None)
        return normed if normed is not None else self._norm(hidden, "model.norm")

    def head_logits(self, features: torch.Tensor) -> torch.Tensor:
        """LM head alone (no norm) on feature rows; fp32 ``[n, V]``.  EAGLE heads borrow the target
        model's vocabulary projection this way (reference: ``cpp/serve/model.cc`` ``GetLogits``)."""
        c = self.cfg
        head = self.p.linears.get("lm_head")
        if head is None:
            emb = self.p.linears.get("model.embed_tokens")
            if emb is not None and emb.kind == "q4" and features.is_cuda and not emb.device_layout:
                head = self._tied_head = getattr(self, "_tied_head", None) or emb.to(features.device)
            else:
                head = emb if emb is not None else ops.dense_weight(self.p.tensors["model.embed_tokens.weight"])
        lg = ops.linear(features.contiguous(), head, out_dtype=torch.float32)
        if "logit_scale" in c.extra:
            lg = lg * c.extra["logit_scale"]
        if c.final_logit_softcap > 0:
            lg = torch.tanh(lg / c.final_logit_softcap) * c.final_logit_softcap
        return lg

    def fuse_embed_hidden(self, embed: torch.Tensor, features: torch.Tensor) -> torch.Tensor:
        """EAGLE input: ``fc([token embedding ; feature of the previous position])``."""
        x = torch.cat([embed, features.to(embed.dtype)], dim=-1).contiguous()
        return ops.linear(x, self.p.linears["model.fc"])

    def medusa_logits(self, features: torch.Tensor, head: int) -> torch.Tensor:
        """Logits of Medusa head ``head`` on feature rows ``[n, H]``; fp32 ``[n, V]``."""
        m = self.cfg.extra["medusa"]
        x = features.to(self.dtype).contiguous()
        for j in range(int(m["num_layers"])):
            y = ops.linear(x, self.p.linears[f"medusa_head.{head}.{j}.linear"])
            x = x + torch.nn.functional.silu(y.float()).to(x.dtype)
        return ops.linear(x, self.p.linears[f"medusa_head.{head}.{int(m['num_layers'])}"], out_dtype=torch.float32)

    def logits(self, hidden: torch.Tensor, rows: Optional[torch.Tensor]) -> torch.Tensor:
        """Final norm + lm_head on the selected rows of the residual stream; fp32 ``[n, V]``."""
        c = self.cfg
        normed = getattr(self, "_final_normed", None)
        if normed is None:
            src = hidden if rows is None else ops.row_gather(hidden, rows)
            h = self._norm(src, "model.norm")
        else:
            h = normed if rows is None else ops.row_gather(normed, rows)
        self._final_normed = None
        head = self.p.linears.get("lm_head")
        if head is None:
            emb = self.p.linears.get("model.embed_tokens")
            if emb is not None and emb.kind == "q4" and h.is_cuda and not emb.device_layout:
                head = self._tied_head = getattr(self, "_tied_head", None) or emb.to(h.device)
            else:
                head = emb if emb is not None else ops.dense_weight(self.p.tensors["model.embed_tokens.weight"])
        lg = ops.linear(h, head, out_dtype=torch.float32)
        if "logit_scale" in c.extra:
            lg = lg * c.extra["logit_scale"]
        if c.final_logit_softcap > 0:
            lg = torch.tanh(lg / c.final_logit_softcap) * c.final_logit_softcap
        return lg


# ---------------------------------------------------------------------------- parameter creation
def param_specs(cfg: ModelConfig) -> Dict[str, tuple]:
    """Full (unsharded) parameter shapes in MLC naming: name -> (shape, kind), kind in
    {"linear", "embedding", "norm", "bias", "experts", "router", "pos"}."""
    h, inter = cfg.hidden_size, cfg.intermediate_size
    hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    medusa = cfg.extra.get("medusa")
    if medusa:
        specs = {}
        for i in range(int(medusa["num_heads"])):
            for j in range(int(medusa["num_layers"])):
                specs[f"medusa_head.{i}.{j}.linear.weight"] = ((h, h), "linear")
                specs[f"medusa_head.{i}.{j}.linear.bias"] = ((h,), "bias")
            specs[f"medusa_head.{i}.{int(medusa['num_layers'])}.weight"] = ((cfg.vocab_size, h), "linear")
        return specs
    if cfg.extra.get("rwkv"):
        specs = {"model.embeddings.weight": ((cfg.vocab_size, h), "pos"),
                 "model.ln_out.weight": ((h,), "norm"), "model.ln_out.bias": ((h,), "bias"),
                 "head.weight": ((cfg.vocab_size, h), "linear")}
        nh, hs = h // cfg.head_dim, cfg.head_dim
        for i in range(cfg.num_hidden_layers):
            p = f"model.blocks.{i}."
            for ln in (["pre_ln"] if i == 0 else []) + ["ln1", "ln2"]:
                specs[p + ln + ".weight"] = ((h,), "norm")
                specs[p + ln + ".bias"] = ((h,), "bias")
            a = p + "attention."
            v6 = int(cfg.extra["rwkv"]) == 6
            specs[a + "time_faaaa"] = ((nh, hs), "f32")
            if v6:
                dm, dd = int(cfg.extra["time_mix_extra_dim"]), int(cfg.extra["time_decay_extra_dim"])
                specs[a + "time_decay"] = ((h,), "f32")       # raw; the decay is computed per token
                for n_ in "xwkvrg":
                    specs[a + f"time_maa_{n_}"] = ((h,), "pos")
                specs[a + "time_maa_w1"] = ((h, 5 * dm), "f32")
                specs[a + "time_maa_w2"] = ((5, dm, h), "f32")
                specs[a + "time_decay_w1"] = ((h, dd), "f32")
                specs[a + "time_decay_w2"] = ((dd, h), "f32")
            else:
                specs[a + "time_decay"] = ((nh, hs), "f32")   # already exp(-exp(.)) of the checkpoint value
            for n_ in ("gate", "key", "value", "receptance"):
                if not v6:
                    specs[a + f"time_mix_{n_}"] = ((h,), "pos")
                specs[a + n_ + ".weight"] = ((h, h), "linear")
            specs[a + "output.weight"] = ((h, h), "linear")
            specs[a + "ln_x.weight"] = ((h,), "norm")
            specs[a + "ln_x.bias"] = ((h,), "bias")
            f = p + "feed_forward."
            if v6:
                specs[f + "time_maa_k"] = ((h,), "pos")
                specs[f + "time_maa_r"] = ((h,), "pos")
            else:
                specs[f + "time_mix_key"] = ((h,), "pos")
                specs[f + "time_mix_receptance"] = ((h,), "pos")
            specs[f + "key.weight"] = ((inter, h), "linear")
            specs[f + "receptance.weight"] = ((h, h), "linear")
            specs[f + "value.weight"] = ((h, inter), "linear")
        return specs
    eagle = bool(cfg.extra.get("eagle"))
    specs: Dict[str, tuple] = {"model.embed_tokens.weight": ((cfg.vocab_size, h), "embedding")}
    if eagle:
        specs["model.fc.weight"] = ((h, 2 * h), "linear")
        if cfg.extra.get("eagle_fc_bias", True):
            specs["model.fc.bias"] = ((h,), "bias")
    if cfg.position_embedding == "learned":
        specs["model.embed_positions.weight"] = ((cfg.context_window_size, h), "pos")
    ln = cfg.norm_type == "layernorm" and not cfg.extra.get("norm_no_affine")
    ln_bias = ln and not cfg.extra.get("norm_no_bias")

    def norm(name, dim=h):
        if cfg.norm_type == "rms" or ln:
            specs[name + ".weight"] = ((dim,), "norm")
        if ln_bias:
            specs[name + ".bias"] = ((dim,), "bias")

    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        if not cfg.extra.get("no_pre_norm") and not (eagle and i == 0):
            norm(p + "input_layernorm")
        mla = cfg.extra.get("mla")
        linear_layer = bool(cfg.extra.get("gdn")) and cfg.layer_attn_kinds[i] == "linear"
        if mla:
            qk = mla["qk_nope_head_dim"] + mla["qk_rope_head_dim"]
            if mla.get("q_lora_rank"):
                specs[p + "self_attn.q_a_proj.weight"] = ((mla["q_lora_rank"], h), "linear")
                specs[p + "self_attn.q_a_layernorm.weight"] = ((mla["q_lora_rank"],), "norm")
                specs[p + "self_attn.q_b_proj.weight"] = ((hq * qk, mla["q_lora_rank"]), "linear")
            else:
                specs[p + "self_attn.q_proj.weight"] = ((hq * qk, h), "linear")
            specs[p + "self_attn.kv_a_proj_with_mqa.weight"] = ((mla["kv_lora_rank"] + mla["qk_rope_head_dim"], h), "linear")
            specs[p + "self_attn.kv_a_layernorm.weight"] = ((mla["kv_lora_rank"],), "norm")
            specs[p + "self_attn.kv_b_proj.weight"] = ((hq * (mla["qk_nope_head_dim"] + mla["v_head_dim"]),
                                                        mla["kv_lora_rank"]), "linear")
            specs[p + "self_attn.o_proj.weight"] = ((h, hq * mla["v_head_dim"]), "linear")
        elif linear_layer:
            # gated delta-rule mixer: [q; k; v] and the output gate z in one projection, the per-head
            # write strength / decay inputs (b, a) in a second, unquantised one
            g = cfg.extra["gdn"]
            kd, vd = g["num_key_heads"] * g["key_head_dim"], g["num_value_heads"] * g["value_head_dim"]
            la = p + "linear_attn."
            specs[la + "in_proj_qkvz.weight"] = ((2 * kd + 2 * vd, h), "linear")
            specs[la + "in_proj_ba.weight"] = ((2 * g["num_value_heads"], h), "router")
            specs[la + "conv1d.weight"] = ((2 * kd + vd, g["conv_kernel"]), "f32")
            specs[la + "dt_bias"] = ((g["num_value_heads"],), "f32")
            specs[la + "A_log"] = ((g["num_value_heads"],), "f32")
            specs[la + "norm.weight"] = ((g["value_head_dim"],), "f32")
            specs[la + "out_proj.weight"] = ((h, vd), "linear")
        else:
            specs[p + "self_attn.qkv_proj.weight"] = (((hq + 2 * hkv) * d, h), "linear")
            if cfg.extra.get("attn_output_gate"):
                specs[p + "self_attn.gate_proj.weight"] = ((hq * d, h), "linear")
            if cfg.attention_bias:
                specs[p + "self_attn.qkv_proj.bias"] = (((hq + 2 * hkv) * d,), "bias")
            specs[p + "self_attn.o_proj.weight"] = ((h, hq * d), "linear")
        if cfg.attention_out_bias:
            specs[p + "self_attn.o_proj.bias"] = ((h,), "bias")
        if cfg.qk_norm and not linear_layer:
            full = bool(cfg.extra.get("qk_norm_full"))
            specs[p + "self_attn.q_norm.weight"] = ((hq * d if full else d,), "norm")
            specs[p + "self_attn.k_norm.weight"] = ((hkv * d if full else d,), "norm")
        if not (cfg.parallel_residual and cfg.shared_input_norm):
            norm(p + "post_attention_layernorm")
        if cfg.post_attention_norm and not cfg.extra.get("no_pre_norm"):
            norm(p + "pre_feedforward_layernorm")
        if cfg.post_mlp_norm:
            norm(p + "post_feedforward_layernorm")
        if cfg.is_moe_layer(i):
            e, mi = cfg.num_experts, cfg.moe_intermediate_size
            specs[p + "moe.gate.weight"] = ((e, h), "router")
            specs[p + "moe.e1_e3.weight"] = ((e, 2 * mi, h), "experts")
            specs[p + "moe.e2.weight"] = ((e, h, mi), "experts")
            if cfg.shared_expert_intermediate_size > 0:
                si = cfg.shared_expert_intermediate_size
                specs[p + "moe.shared_expert.gate_up_proj.weight"] = ((2 * si, h), "linear")
                specs[p + "moe.shared_expert.down_proj.weight"] = ((h, si), "linear")
                if cfg.shared_expert_gate:
                    specs[p + "moe.shared_expert_gate.weight"] = ((1, h), "router")
        elif cfg.gated_mlp:
            specs[p + "mlp.gate_up_proj.weight"] = ((2 * inter, h), "linear")
            specs[p + "mlp.down_proj.weight"] = ((h, inter), "linear")
            if cfg.mlp_bias:
                specs[p + "mlp.gate_up_proj.bias"] = ((2 * inter,), "bias")
                specs[p + "mlp.down_proj.bias"] = ((h,), "bias")
        else:
            specs[p + "mlp.up_proj.weight"] = ((inter, h), "linear")
            specs[p + "mlp.down_proj.weight"] = ((h, inter), "linear")
            if cfg.mlp_bias:
                specs[p + "mlp.up_proj.bias"] = ((inter,), "bias")
                specs[p + "mlp.down_proj.bias"] = ((h,), "bias")
    if not eagle:
        norm("model.norm")
    if not cfg.tie_word_embeddings:
        specs["lm_head.weight"] = ((cfg.vocab_size, h), "linear")
        if cfg.lm_head_bias:
            specs["lm_head.bias"] = ((cfg.vocab_size,), "bias")
    return specs


def shard_rows(name: str, cfg: ModelConfig, tp: int, rank: int, full_rows: int):
    """Row (output-feature) index ranges of `name` kept by `rank`; None = replicated / column-sharded.
    Follows the reference's ShardSingleDim segments (support/tensor_parallel.py:36-97): qkv_proj is
    split per segment [q, k, v], gate_up_proj per segment [gate, up]."""
    d = cfg.head_dim
    if name.endswith("self_attn.qkv_proj"):
        segs = [cfg.num_attention_heads * d, cfg.num_key_value_heads * d, cfg.num_key_value_heads * d]
    elif name.endswith("gate_up_proj"):
        segs = [full_rows // 2, full_rows // 2]
    elif name.endswith("mlp.up_proj"):
        segs = [full_rows]
    elif cfg.extra.get("gdn") and name.endswith("linear_attn.in_proj_qkvz"):
        # gated delta-rule mixer: key heads and value heads are split over the ranks together
        g = cfg.extra["gdn"]
        kd, vd = g["num_key_heads"] * g["key_head_dim"], g["num_value_heads"] * g["value_head_dim"]
        segs = [kd, kd, vd, vd]
    elif name.endswith("self_attn.gate_proj"):
        segs = [full_rows]  # output gate of the attention heads: split like the heads
    elif cfg.extra.get("rwkv") and name.endswith(("attention.receptance", "attention.key", "attention.value",
                                                   "attention.gate", "feed_forward.key")):
        # recurrent models: a rank keeps whole heads of the time-mix projections and a slice of the channel-mix
        # width (reference: the shard strategies of python/mlc_llm/model/rwkv6/rwkv6_model.py)
        segs = [full_rows]
    elif cfg.extra.get("mla") and name.endswith(("self_attn.q_b_proj", "self_attn.q_proj", "self_attn.kv_b_proj")):
        # latent attention: the per-head up-projections are head-major, so a rank keeps the rows of its heads;
        # the down-projections to the latents (q_a, kv_a) stay whole on every rank
        segs = [full_rows]
    else:
        return None
    out, off = [], 0
    for s in segs:
        per = s // tp
        out.append((off + rank * per, off + (rank + 1) * per))
        off += s
    return out


def column_sharded(name: str) -> bool:
    return name.endswith(("self_attn.o_proj", "down_proj", "linear_attn.out_proj")) or (
        name.startswith("model.blocks.") and name.endswith(("attention.output", "feed_forward.value")))  # RWKV
