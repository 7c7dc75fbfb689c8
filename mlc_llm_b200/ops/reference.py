"""Plain PyTorch fp32 restatement of every operator.

These functions are (a) the CPU execution path of the engine, so the whole serving stack runs
without a GPU, and (b) the numerical oracle every CUDA kernel is tested against.  They use the same
tensor layouts as the kernels (paged KV ``[pages, 2, hkv, page, d]``, fused ``qkv`` rows, packed
int4 words) so model code is identical on both devices.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from .. import quantization as Q


# --------------------------------------------------------------------------- linear
def linear_dense(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or x.dtype)


def linear_q4(x: torch.Tensor, qw_artifact: torch.Tensor, qs: torch.Tensor,
              quant: Q.Quantization, bias: Optional[torch.Tensor] = None,
              out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    w = Q.group_dequantize(qw_artifact, qs, quant, k=x.shape[-1])
    return linear_dense(x, w, bias, out_dtype)


# --------------------------------------------------------------------------- norms / activations
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, w_offset: float = 0.0) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * inv * (w.float() + w_offset)).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float,
                w_offset: float = 0.0) -> torch.Tensor:
    """residual += x (rounded to the storage dtype), returns rmsnorm(residual)."""
    s = (x.float() + residual.float()).to(residual.dtype)
    residual.copy_(s)
    return rmsnorm(residual, w, eps, w_offset)


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return torch.nn.functional.layer_norm(
        x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps).to(x.dtype)


def act_mul(x: torch.Tensor, act: str = "silu") -> torch.Tensor:
    inter = x.shape[-1] // 2
    g, u = x[..., :inter].float(), x[..., inter:].float()
    if act == "silu":
        a = g * torch.sigmoid(g)
    else:
        a = torch.nn.functional.gelu(g, approximate="tanh")
    a = a.to(x.dtype).float()
    return (a * u).to(x.dtype)


# --------------------------------------------------------------------------- RoPE
def rope_inv_freq(rot_dim: int, theta: float, scaling: Optional[dict] = None) -> torch.Tensor:
    """Inverse frequencies with optional ``llama3`` scaling (model/llama/llama_model.py:52-58)."""
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv
        smooth = (orig / wavelen - low) / (high - low)
        scaled = torch.where(
            wavelen > orig / low, inv / factor,
            torch.where(wavelen < orig / high, inv, (1 - smooth) * inv / factor + smooth * inv))
        inv = scaled
    elif scaling and scaling.get("rope_type", scaling.get("type")) == "linear":
        inv = inv / float(scaling["factor"])
    elif scaling and scaling.get("rope_type", scaling.get("type")) == "yarn":
        # YaRN: bands that turn more than beta_fast times inside the original window keep their frequency,
        # bands that turn less than beta_slow times are slowed by `factor`, a linear ramp in between
        factor = float(scaling["factor"])
        orig = float(scaling.get("original_max_position_embeddings") or 0) or 4096.0
        fast, slow = float(scaling.get("beta_fast") or 32), float(scaling.get("beta_slow") or 1)

        def band_of(turns: float) -> float:
            return rot_dim * math.log(orig / (turns * 2 * math.pi)) / (2 * math.log(theta))

        low, high = band_of(fast), band_of(slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, rot_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rot_dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        inv = (inv / factor) * ramp + inv * (1 - ramp)
    elif scaling and scaling.get("rope_type", scaling.get("type")) in ("longrope", "su"):
        # per-band divisors: the long set once the context exceeds the window the model was trained on
        orig = int(scaling.get("original_max_position_embeddings") or 0)
        cur = int(scaling.get("max_position_embeddings") or 0)
        ext = scaling["long_factor"] if (orig and cur > orig) else scaling["short_factor"]
        inv = inv / torch.tensor(ext, dtype=torch.float64)
    elif scaling and scaling.get("rope_type", scaling.get("type", "default")) not in ("default", "mrope", None):
        import logging  # pylint: disable=import-outside-toplevel

        logging.getLogger(__name__).warning("rotary scaling %r is not implemented; plain frequencies are used",
                                            scaling.get("rope_type", scaling.get("type")))
    return inv.to(torch.float32)


def _yarn_mscale(factor: float, mscale: float = 1.0) -> float:
    return 1.0 if factor <= 1 else 0.1 * mscale * math.log(factor) + 1.0


def rope_attention_factor(scaling: Optional[dict]) -> float:
    """Scale applied to cos / sin (hence to q and k) by the rotary variants that stretch the context:
    YaRN ``0.1 ln(factor) + 1`` (or the ratio of its two ``mscale`` forms), LongRoPE
    ``sqrt(1 + ln(scale) / ln(original window))``; 1 otherwise."""
    if not scaling:
        return 1.0
    kind = scaling.get("rope_type", scaling.get("type"))
    if scaling.get("attention_factor") is not None and kind in ("yarn", "longrope", "su"):
        return float(scaling["attention_factor"])
    if kind == "yarn":
        factor = float(scaling["factor"])
        ms, ms_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
        if ms and ms_all:
            return _yarn_mscale(factor, float(ms)) / _yarn_mscale(factor, float(ms_all))
        return _yarn_mscale(factor)
    if kind in ("longrope", "su"):
        orig = int(scaling.get("original_max_position_embeddings") or 0)
        cur = int(scaling.get("max_position_embeddings") or 0)
        if not orig or cur <= orig:
            return 1.0
        return math.sqrt(1.0 + math.log(cur / orig) / math.log(orig))
    return 1.0


def rope_append(qkv: torch.Tensor, kv_pages: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor,
                inv_freq: Optional[torch.Tensor], hq: int, hkv: int, d: int, rot_dim: int, page: int,
                attn_factor: float = 1.0) -> None:
    """Rotate q and k heads of ``qkv [T, (hq+2hkv)*d]`` in place and append k, v to their slots."""
    t = qkv.shape[0]
    if t == 0:
        return
    heads = qkv.view(t, hq + 2 * hkv, d)
    if inv_freq is not None and rot_dim > 0:
        ang = pos.to(torch.float32).unsqueeze(-1) * inv_freq.to(qkv.device).unsqueeze(0)  # [T, rot/2]
        cos = (torch.cos(ang) * attn_factor).unsqueeze(1)
        sin = (torch.sin(ang) * attn_factor).unsqueeze(1)
        half = rot_dim // 2
        qk = heads[:, : hq + hkv, :rot_dim].float()
        a, b = qk[..., :half], qk[..., half:]
        lo, hi = a * cos - b * sin, b * cos + a * sin  # both before writing: qk aliases heads in fp32
        heads[:, : hq + hkv, :half] = lo.to(qkv.dtype)
        heads[:, : hq + hkv, half:rot_dim] = hi.to(qkv.dtype)
    valid = slot >= 0
    if valid.any():
        sl = slot[valid].long()
        pg, off = sl // page, sl % page
        kv_pages[pg, 0, :, off, :] = heads[valid, hq : hq + hkv, :]
        kv_pages[pg, 1, :, off, :] = heads[valid, hq + hkv :, :]


# --------------------------------------------------------------------------- attention
def paged_attention(q: torch.Tensor, kv_pages: torch.Tensor, q_seq: torch.Tensor,
                    q_kvlen: torch.Tensor, page_indptr: torch.Tensor, page_indices: torch.Tensor,
                    hq: int, hkv: int, d: int, page: int, sm_scale: float,
                    q_kvstart: Optional[torch.Tensor] = None, sink: int = 0,
                    tree_mask: Optional[torch.Tensor] = None, softcap: float = 0.0,
                    return_lse: bool = False):
    """``q [T, hq, d]`` (any row stride) attends to the paged KV of its sequence.

    Token ``t`` sees positions ``j < q_kvlen[t]`` with ``j < sink or j >= q_kvstart[t]``, plus, when
    ``tree_mask`` is given, positions ``q_kvlen[t] + b`` for every set bit ``b``.
    """
    t = q.shape[0]
    out = torch.zeros(t, hq, d, dtype=q.dtype, device=q.device)
    lse = torch.full((t, hq), -float("inf"), dtype=torch.float32, device=q.device)
    g = hq // hkv
    for i in range(t):
        b = int(q_seq[i])
        n = int(q_kvlen[i])
        tm = int(tree_mask[i]) if tree_mask is not None else 0
        total = n + (tm.bit_length() if tm else 0)
        if total == 0:
            continue
        pages = page_indices[int(page_indptr[b]) : int(page_indptr[b + 1])].long()
        npg = (total + page - 1) // page
        kv = kv_pages[pages[:npg]]  # [npg, 2, hkv, page, d]
        k = kv[:, 0].permute(1, 0, 2, 3).reshape(hkv, npg * page, d)[:, :total].float()
        v = kv[:, 1].permute(1, 0, 2, 3).reshape(hkv, npg * page, d)[:, :total].float()
        idx = torch.arange(total, device=q.device)
        start = int(q_kvstart[i]) if q_kvstart is not None else 0
        vis = (idx < n) & ((idx < sink) | (idx >= start))
        if tm:
            bits = torch.tensor([(tm >> j) & 1 for j in range(total - n)], dtype=torch.bool,
                                device=q.device)
            vis[n:] = bits
        qi = q[i].float().view(hkv, g, d)
        s = torch.einsum("hgd,hnd->hgn", qi, k) * sm_scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~vis.view(1, 1, -1), -float("inf"))
        lse[i] = torch.logsumexp(s, dim=-1).reshape(hq)
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)
        out[i] = torch.einsum("hgn,hnd->hgd", p, v).reshape(hq, d).to(q.dtype)
    return (out, lse) if return_lse else out


def mla_append(rows: torch.Tensor, cache: torch.Tensor, slot: torch.Tensor, page: int) -> None:
    """``rows [T, D]`` into the slots of a latent cache ``[num_pages, 1, 1, page, D]``; negative slots are skipped."""
    valid = slot >= 0
    if valid.any():
        sl = slot[valid].long()
        cache[sl // page, 0, 0, sl % page, :] = rows[valid].to(cache.dtype)


def mla_attention(q: torch.Tensor, cache: torch.Tensor, q_seq: torch.Tensor, q_kvlen: torch.Tensor,
                  page_indptr: torch.Tensor, page_indices: torch.Tensor, rope: int, rank: int, page: int,
                  sm_scale: float, q_kvstart: Optional[torch.Tensor] = None, sink: int = 0,
                  tree_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Absorbed latent attention: ``q [T, hq, rope + rank]`` against cached rows ``[rope | latent]`` shared by all
    heads; returns the softmax-weighted latents ``[T, hq, rank]``. Visibility as in :func:`paged_attention`."""
    t, hq, d = q.shape
    out = torch.zeros(t, hq, rank, dtype=q.dtype, device=q.device)
    for i in range(t):
        b = int(q_seq[i])
        n = int(q_kvlen[i])
        tm = int(tree_mask[i]) if tree_mask is not None else 0
        total = n + (tm.bit_length() if tm else 0)
        if total == 0:
            continue
        pages = page_indices[int(page_indptr[b]) : int(page_indptr[b + 1])].long()
        npg = (total + page - 1) // page
        rows = cache[pages[:npg], 0, 0].reshape(npg * page, d)[:total].float()
        idx = torch.arange(total, device=q.device)
        start = int(q_kvstart[i]) if q_kvstart is not None else 0
        vis = (idx < n) & ((idx < sink) | (idx >= start))
        if tm:
            vis[n:] = torch.tensor([(tm >> j) & 1 for j in range(total - n)], dtype=torch.bool, device=q.device)
        s = (q[i].float() @ rows.T) * sm_scale
        s = s.masked_fill(~vis.view(1, -1), -float("inf"))
        p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
        out[i] = (p @ rows[:, rope:]).to(q.dtype)
    return out


# --------------------------------------------------------------------------- logits / sampling
def softmax_temperature(logits: torch.Tensor, temperature: torch.Tensor,
                        active_vocab: int = 0) -> torch.Tensor:
    """Reference: attach_softmax_with_temperature.py:43-274 (T ~ 0 spreads mass over the argmax set)."""
    n, v = logits.shape
    lg = logits.float().clone()
    if 0 < active_vocab < v:
        lg[:, active_vocab:] = -float("inf")
    probs = torch.empty_like(lg)
    for i in range(n):
        t = float(temperature[i])
        if t < 1e-5:
            mx = lg[i].max()
            hit = (lg[i] == mx).float()
            probs[i] = hit / hit.sum()
        else:
            probs[i] = torch.softmax(lg[i] / t, dim=-1)
    return probs


def apply_logit_bias(logits, pos2seq, token, bias):
    for r, tk, b in zip(pos2seq.tolist(), token.tolist(), bias.tolist()):
        logits[r, tk] += b


def apply_penalty(logits, pos2seq, token, cnt, penalties):
    """attach_logit_processor.py:156-207: presence/frequency subtract, then repetition scale."""
    for r, tk, c in zip(pos2seq.tolist(), token.tolist(), cnt.tolist()):
        v = float(logits[r, tk]) - (float(penalties[r, 0]) + c * float(penalties[r, 1]))
        rep = float(penalties[r, 2])
        logits[r, tk] = v * rep if v < 0 else v / rep


def apply_bitmask(logits, rows, bitmask):
    v = logits.shape[1]
    idx = torch.arange(v, device=logits.device)
    for r, row in enumerate(rows.tolist()):
        bits = (bitmask[r, idx // 32].to(torch.int64) >> (idx % 32)) & 1
        logits[row, bits == 0] = torch.finfo(torch.float32).min


def top_p_cutoff(p: torch.Tensor, top_p: float, top_k: int = 0):
    """(cutoff value, kept mass): smallest set of largest probs with mass >= top_p (ties kept)."""
    total = float(p.sum())
    v = p.numel()
    if top_p >= 1 - 1e-5 and (top_k <= 0 or top_k >= v):
        return 0.0, total
    sp, _ = torch.sort(p, descending=True)
    cs = torch.cumsum(sp.double(), 0)
    if top_p >= 1 - 1e-5:
        kp = v
    else:
        kp = int(torch.searchsorted(cs, torch.tensor(top_p * total, dtype=torch.float64)).item()) + 1
        kp = min(kp, v)
    if 0 < top_k < v:
        kp = min(kp, top_k)
    cutoff = float(sp[kp - 1])
    kept = p >= cutoff
    return cutoff, float(p[kept].sum())


def sample(probs: torch.Tensor, rows: Optional[torch.Tensor], uniform: torch.Tensor,
           top_p: Optional[torch.Tensor], top_k: Optional[torch.Tensor] = None):
    """Index-order inverse-CDF sampling over the top-p / top-k set; returns (tokens, probs)."""
    n = uniform.shape[0]
    toks = torch.zeros(n, dtype=torch.int32)
    outp = torch.zeros(n, dtype=torch.float32)
    for r in range(n):
        row = int(rows[r]) if rows is not None else r
        p = probs[row].float().cpu()
        tp = float(top_p[r]) if top_p is not None else 1.0
        tk = int(top_k[r]) if top_k is not None else 0
        if tp <= 0:
            toks[r] = int(torch.argmax(p))
            outp[r] = 1.0
            continue
        cutoff, mass = top_p_cutoff(p, tp, tk)
        kept = torch.where(p >= cutoff, p, torch.zeros_like(p))
        cdf = torch.cumsum(kept.double(), 0)
        target = float(uniform[r]) * mass
        idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
        if idx >= p.numel():
            idx = int(torch.nonzero(kept > 0)[-1])
        toks[r] = idx
        outp[r] = float(p[idx]) / mass if mass > 0 else 0.0
    return toks, outp


def renorm_top_p(probs: torch.Tensor, rows: Optional[torch.Tensor], top_p: torch.Tensor) -> None:
    for r in range(top_p.shape[0]):
        row = int(rows[r]) if rows is not None else r
        p = probs[row]
        cutoff, mass = top_p_cutoff(p.float().cpu(), float(top_p[r]))
        probs[row] = torch.where(p >= cutoff, p / mass, torch.zeros_like(p))


def take_probs(probs, rows, token, k):
    n = token.shape[0]
    outp = torch.zeros(n)
    tp = torch.zeros(n, max(k, 1))
    ti = torch.zeros(n, max(k, 1), dtype=torch.int32)
    for r in range(n):
        row = int(rows[r]) if rows is not None else r
        outp[r] = probs[row, int(token[r])]
        if k:
            v, i = torch.topk(probs[row].float(), k)
            tp[r, :k], ti[r, :k] = v, i.to(torch.int32)
    return outp, tp[:, :k], ti[:, :k]


def verify_tree(draft_probs, draft_tokens, model_probs, first_child, next_sibling, uniform,
                parent_ptr) -> None:
    """op/batch_spec_verify.py:8-175: accept a child when p >= u * q (and p > 0), otherwise replace the
    parent distribution by normalise(max(p - q, 0)) and try the next sibling."""
    for b in range(parent_ptr.shape[0]):
        parent = int(parent_ptr[b])
        child = int(first_child[parent])
        while child >= 0:
            tok = int(draft_tokens[child])
            p = float(model_probs[parent, tok])
            qv = float(draft_probs[child, tok])
            if p > 0.0 and p >= float(uniform[child]) * qv:  # p > 0: see the kernel's note on q == 0
                parent, child = child, int(first_child[child])
            else:
                r = torch.clamp(model_probs[parent] - draft_probs[child], min=0)
                s = r.sum()
                model_probs[parent] = r / s if s > 0 else r
                child = int(next_sibling[child])
        parent_ptr[b] = parent


# --------------------------------------------------------------------------- MoE
def moe_topk_softmax(gate_logits: torch.Tensor, k: int, norm_topk: bool = True):
    """Top-k over raw logits, softmax over the selected k in fp32 (op/moe_misc.py:135-235)."""
    vals, idx = torch.topk(gate_logits.float(), k, dim=-1)
    w = torch.softmax(vals, dim=-1) if norm_topk else vals
    return w, idx.to(torch.int32)


def moe_softmax_topk(gate_logits: torch.Tensor, k: int, renorm: bool):
    """Softmax over all experts then top-k (qwen-moe style), optional renormalisation."""
    p = torch.softmax(gate_logits.float(), dim=-1)
    vals, idx = torch.topk(p, k, dim=-1)
    if renorm:
        vals = vals / vals.sum(dim=-1, keepdim=True)
    return vals, idx.to(torch.int32)


def moe_ffn(x, w13, w2, weights, experts, act: str = "silu"):
    """x [T, H]; w13 [E, 2I, H]; w2 [E, H, I]; weights/experts [T, k]. Returns [T, H]."""
    t, h = x.shape
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    for e in range(w13.shape[0]):
        sel = (experts == e)
        tok, slot = torch.nonzero(sel, as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        h1 = linear_dense(xe, w13[e])
        a = act_mul(h1, act)
        y = linear_dense(a, w2[e]).float()
        out.index_add_(0, tok, y * weights[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)
