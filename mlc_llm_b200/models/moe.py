"""Mixture-of-experts block: router -> expert-major permutation -> grouped GEMMs -> weighted combine.

Reference: ``model/mixtral/mixtral_model.py:64-117`` (softmax-top-k routing, ``e1_e3`` / ``e2`` expert
matmuls, scatter back and weighted sum) and ``model/qwen2_moe`` / ``qwen3_moe`` (shared expert,
optional renormalisation).  Under tensor parallelism the experts are sharded on their intermediate
dimension as in the reference (``mixtral_model.py:144-145``); with ``expert_parallel`` whole experts
live on different ranks and tokens travel through the all-to-all in ``parallel/expert.py``.
"""

from __future__ import annotations

import torch

from .. import ops


def _group_limited_router(logits: torch.Tensor, k: int, n_group: int, topk_group: int, renorm: bool):
    """DeepSeek-V2 routing: softmax over all experts, keep the ``topk_group`` expert groups with the
    best single score, then the top ``k`` experts inside them (reference: ``op/moe_misc.py:238-368``)."""
    t, e = logits.shape
    if logits.is_cuda and k <= 8 and n_group <= 32 and e % n_group == 0:
        from ..ops._lib import DTYPE_CODE, check, lib, ptr, stream_ptr  # pylint: disable=import-outside-toplevel
        import ctypes  # pylint: disable=import-outside-toplevel

        lg = logits.contiguous()
        w = torch.empty(t, k, dtype=torch.float32, device=lg.device)
        idx = torch.empty(t, k, dtype=torch.int32, device=lg.device)
        rc = lib().mlcb_moe_router_grouped(ptr(lg), ptr(w), ptr(idx), ctypes.c_int(t), ctypes.c_int(e), ctypes.c_int(k),
                                           ctypes.c_int(n_group), ctypes.c_int(topk_group),
                                           ctypes.c_int(1 if renorm else 0), ctypes.c_int(DTYPE_CODE[lg.dtype]),
                                           stream_ptr())
        check(rc, "mlcb_moe_router_grouped")
        return w, idx
    probs = torch.softmax(logits.float(), dim=-1)
    group_best = probs.view(t, n_group, e // n_group).max(dim=-1).values
    keep = torch.zeros_like(group_best).scatter_(1, torch.topk(group_best, topk_group, dim=-1).indices, 1.0)
    masked = probs.masked_fill(keep.unsqueeze(-1).expand(t, n_group, e // n_group).reshape(t, e) == 0, 0.0)
    w, idx = torch.topk(masked, k, dim=-1)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.float().contiguous(), idx.to(torch.int32).contiguous()  # fp32 weights, like ops.moe_router


def _llama4_moe(model, li: int, h: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
    """Llama-4 routing: top-k over the raw logits; the *input* of each chosen expert is scaled by the sigmoid of
    its logit, the expert outputs are summed unweighted, and a shared expert is added (reference:
    ``python/mlc_llm/model/llama4/llama4_model.py:363-410``)."""
    c = model.cfg
    if c.expert_parallel and model.comm is not None and model.tp > 1:
        raise NotImplementedError("expert parallelism is not available for the Llama-4 router")
    pre = f"model.layers.{li}.moe."
    t, k = h.shape[0], c.num_experts_per_tok
    top_v, idx = torch.topk(logits.float(), k, dim=-1)
    scores = torch.sigmoid(top_v)                                         # [T, k]
    experts = idx.to(torch.int32).contiguous()
    offsets, sorted_pos, src_token = ops.moe_permute(experts, c.num_experts)
    row_scale = torch.empty(t * k, dtype=torch.float32, device=h.device)
    row_scale[sorted_pos.long()] = scores.reshape(-1)
    xp = (ops.row_gather(h, src_token).float() * row_scale.unsqueeze(-1)).to(h.dtype)
    h1 = ops.grouped_linear(xp, model.p.linears[pre + "e1_e3"], offsets)
    y = ops.grouped_linear(ops.act_mul(h1, "silu"), model.p.linears[pre + "e2"], offsets)
    ones = torch.ones(t, k, dtype=torch.float32, device=h.device)
    out = ops.moe_combine(y, ones, sorted_pos, None)
    g = ops.linear(h, model.p.linears[pre + "shared_expert.gate_up_proj"])
    return out + ops.linear(ops.act_mul(g, "silu"), model.p.linears[pre + "shared_expert.down_proj"])


def moe_block(model, li: int, h: torch.Tensor) -> torch.Tensor:
    c = model.cfg
    pre = f"model.layers.{li}.moe."
    t, hidden = h.shape
    k = c.num_experts_per_tok
    gate_w = model.p.tensors[pre + "gate.weight"]
    logits = ops.linear(h, ops.dense_weight(gate_w))
    if c.moe_router == "llama4_sigmoid":
        return _llama4_moe(model, li, h, logits)
    renorm = c.norm_topk_prob if c.moe_router == "softmax_topk" else True
    if c.extra.get("topk_method") == "group_limited_greedy" and c.extra.get("n_group", 1) > 1:
        weights, experts = _group_limited_router(logits, k, c.extra["n_group"], c.extra["topk_group"], renorm)
    else:
        weights, experts = ops.moe_router(logits, k, renorm)
    scale = float(c.extra.get("routed_scaling_factor", 1.0))
    if scale != 1.0:
        weights = weights * scale
    w13 = model.p.linears[pre + "e1_e3"]
    w2 = model.p.linears[pre + "e2"]
    if c.expert_parallel and model.comm is not None and model.tp > 1:
        from ..parallel.expert import expert_parallel_ffn  # pylint: disable=import-outside-toplevel

        out = expert_parallel_ffn(model, h, weights, experts, w13, w2)
        model._mlp_complete = True  # every expert ran whole on some rank: nothing to all-reduce
    else:
        offsets, sorted_pos, src_token = ops.moe_permute(experts, c.num_experts)
        xp = ops.row_gather(h, src_token)
        h1 = ops.grouped_linear(xp, w13, offsets)
        a = ops.act_mul(h1, "silu" if c.hidden_act == "silu" else "gelu")
        y = ops.grouped_linear(a, w2, offsets)
        out = ops.moe_combine(y, weights, sorted_pos, None)
    if c.shared_expert_intermediate_size > 0:
        g = ops.linear(h, model.p.linears[pre + "shared_expert.gate_up_proj"])
        s = ops.linear(ops.act_mul(g, "silu"), model.p.linears[pre + "shared_expert.down_proj"])
        if c.shared_expert_gate:
            sg = ops.linear(h, ops.dense_weight(model.p.tensors[pre + "shared_expert_gate.weight"]))
            s = (torch.sigmoid(sg.float()) * s.float()).to(s.dtype)
        if getattr(model, "_mlp_complete", False):
            s = model._reduce(s)  # the shared expert stays sharded over its width
        out = out + s
    return out
