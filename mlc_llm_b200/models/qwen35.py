"""Qwen3.5 hybrid decoder: gated delta-rule ("linear attention") layers with a per-sequence recurrent
state, interleaved with softmax-attention layers on the paged KV cache.

Reference: ``python/mlc_llm/model/qwen35/qwen35_model.py`` (GatedDeltaNet layers holding a convolution
state and a recurrent state in an RNN-state object next to the paged KV cache of the attention layers).

A linear layer does, per token t and value head h (state ``S`` is ``[key_dim, value_dim]``)::

    [q; k; v] = silu(causal_conv1d([q; k; v] projections, kernel 4))      q, k L2-normalised, q / sqrt(key_dim)
    g = -exp(A_log) * softplus(a + dt_bias)          beta = sigmoid(b)
    S  <- S * exp(g)
    S  <- S + k (x) (beta * (v - S^T k))             # delta rule: move the value stored under k towards v
    o  = S^T q
    y  = out_proj( rmsnorm(o) * weight * silu(z) )

An attention layer is Qwen3 attention (per-head q / k RMS norm, a quarter of every head rotated) whose
context is multiplied by ``sigmoid(gate)``, a second query-sized projection of the layer input.

Only the attention layers own KV pages; the recurrent state lives in two slot tensors indexed by a
sequence-id map, so a decode step over many sequences is one batched update.
"""

from __future__ import annotations

import collections
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from .transformer import BatchInfo, DecoderModel

STATE_SLOTS = 256  # sequences whose recurrent state is kept; the least recently used one is dropped
FIRST_SLOTS = 16   # the slot tensors start this large and double on demand (a slot is megabytes per layer)


def gated_delta_step(state: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     g: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """One token of the recurrence for a batch. ``state`` [B, H, dk, dv] fp32 (updated in place),
    ``q`` / ``k`` [B, H, dk] (normalised, q scaled), ``v`` [B, H, dv], ``g`` / ``beta`` [B, H].
    Returns the read-out [B, H, dv]."""
    state.mul_(g.exp().unsqueeze(-1).unsqueeze(-1))
    stored = torch.einsum("bhkv,bhk->bhv", state, k)
    delta = (v - stored) * beta.unsqueeze(-1)
    state.add_(k.unsqueeze(-1) * delta.unsqueeze(-2))
    return torch.einsum("bhkv,bhk->bhv", state, q)


def _gdn_step_kernel(rec_all: torch.Tensor, slots, q, k, v, g, beta, out: torch.Tensor, rows) -> bool:
    """The decode step as one kernel, in place on the state pool ``rec_all [slots, H, dk, dv]`` (no gather /
    scatter of the states). Returns False when the kernel does not apply (CPU, other head sizes)."""
    if not rec_all.is_cuda or rec_all.dtype != torch.float32 or not rec_all.is_contiguous() \
            or q.shape[-1] not in (64, 128) or v.shape[-1] % 32 or q.shape[-1] * v.shape[-1] > 128 * 128:
        return False
    import ctypes  # pylint: disable=import-outside-toplevel

    from ..ops._lib import check, lib, ptr, stream_ptr  # pylint: disable=import-outside-toplevel

    b, h, dk = q.shape
    dv = v.shape[-1]
    slots_t = torch.as_tensor(slots, device=rec_all.device).to(torch.int32).contiguous()
    res = torch.empty(b, h, dv, dtype=torch.float32, device=rec_all.device)
    rc = lib().mlcb_gdn_step(ptr(rec_all), ptr(slots_t), ptr(q.float().contiguous()), ptr(k.float().contiguous()),
                             ptr(v.float().contiguous()), ptr(g.float().contiguous()), ptr(beta.float().contiguous()),
                             ptr(res), ctypes.c_int(b), ctypes.c_int(h), ctypes.c_int(dk), ctypes.c_int(dv),
                             stream_ptr())
    if rc < 0:
        return False
    check(rc, "mlcb_gdn_step")
    out[rows] = res
    return True


def gated_delta_chunk(state: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                      g: torch.Tensor, beta: torch.Tensor, chunk: int = 64) -> torch.Tensor:
    """The same recurrence for ``n`` consecutive tokens of one sequence, ``chunk`` tokens per step, as
    matrix products. ``state`` [H, dk, dv] fp32 (updated in place), ``q`` / ``k`` [n, H, dk], ``v`` [n, H, dv],
    ``g`` / ``beta`` [n, H]; returns [n, H, dv].

    Inside a chunk that starts from state ``S0``, with ``G`` the running sum of ``g`` and ``u_i`` the row
    written at token i (``S_i = exp(g_i) S_{i-1} + k_i u_i^T``):

        u_i = beta_i * (v_i - exp(G_i) S0^T k_i - sum_{j<i} exp(G_i - G_j) (k_i . k_j) u_j)
        o_i = exp(G_i) S0^T q_i + sum_{j<=i} exp(G_i - G_j) (q_i . k_j) u_j
        S_end = exp(G_end) S0 + sum_j exp(G_end - G_j) k_j u_j^T

    The first line is a unit-lower-triangular system in ``u``; every exponent is <= 0.
    """
    n = q.shape[0]
    out = torch.empty(n, v.shape[1], v.shape[2], dtype=torch.float32, device=q.device)
    for c0 in range(0, n, chunk):
        c1 = min(n, c0 + chunk)
        qc, kc, vc = (x[c0:c1].transpose(0, 1).float() for x in (q, k, v))          # [H, C, d]
        gc, bc = g[c0:c1].t().float(), beta[c0:c1].t().float()                       # [H, C]
        cum = gc.cumsum(-1)
        rel = cum.unsqueeze(-1) - cum.unsqueeze(-2)                                   # G_i - G_j
        lower = torch.ones(c1 - c0, c1 - c0, dtype=torch.bool, device=q.device).tril()
        decay = torch.where(lower, rel, torch.full_like(rel, float("-inf"))).exp()    # 0 above the diagonal
        grow = cum.exp().unsqueeze(-1)                                                # exp(G_i)
        kk = (kc @ kc.transpose(-1, -2)) * decay * bc.unsqueeze(-1)
        system = torch.eye(c1 - c0, device=q.device) + kk.tril(-1)
        rhs = bc.unsqueeze(-1) * (vc - grow * (kc @ state))
        u = torch.linalg.solve_triangular(system, rhs, upper=False, unitriangular=True)
        out[c0:c1] = (grow * (qc @ state) + ((qc @ kc.transpose(-1, -2)) * decay) @ u).transpose(0, 1)
        tail = (cum[:, -1:] - cum).exp().unsqueeze(-1)                                # exp(G_end - G_j)
        state.mul_(cum[:, -1].exp().view(-1, 1, 1)).add_((kc * tail).transpose(-1, -2) @ u)
    return out


class Qwen35Model(DecoderModel):
    """Hybrid model behind the decoder-model interface of the executor."""

    stateful = True  # per-sequence recurrent state: sequences are told apart by id, no CUDA-graph replay

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        c = self.cfg
        g = c.extra["gdn"]
        # tensor parallelism: a rank keeps `nk / tp` key heads and the `nv / tp` value heads that go with them
        # (projection rows, convolution channels, decay / gate parameters, recurrent state); `out_proj` is split
        # on its input and the caller sums the partial outputs like an attention block's
        self.nk_all, self.nv_all = int(g["num_key_heads"]), int(g["num_value_heads"])
        if self.nk_all % self.tp or self.nv_all % self.tp:
            raise ValueError(f"{self.nk_all} key / {self.nv_all} value heads cannot be split over {self.tp} ranks")
        self.nk, self.nv = self.nk_all // self.tp, self.nv_all // self.tp
        self.rank = self.comm.tp_rank if (self.comm is not None and self.tp > 1) else 0
        self._gdn_params: dict = {}
        self.dk, self.dv = int(g["key_head_dim"]), int(g["value_head_dim"])
        self.kernel = int(g["conv_kernel"])
        self.key_dim, self.value_dim = self.nk * self.dk, self.nv * self.dv
        self.conv_dim = 2 * self.key_dim + self.value_dim
        kinds = c.layer_attn_kinds
        self.attn_layers = [li for li in self.layers if kinds[li] != "linear"]
        self.linear_layers = [li for li in self.layers if kinds[li] == "linear"]
        self._kv_of = {li: i for i, li in enumerate(self.attn_layers)}
        self._lin_of = {li: i for i, li in enumerate(self.linear_layers)}
        self.slot_of: "collections.OrderedDict[int, int]" = collections.OrderedDict()
        self.free_slots: List[int] = []
        self.capacity = 0
        self.conv_state: Optional[torch.Tensor] = None
        self.rec_state: Optional[torch.Tensor] = None
        self._ctx: Optional[dict] = None

    # ------------------------------------------------------------------ caches
    def create_kv_cache(self, num_pages: int, page_size: int = 16) -> None:
        self.page = page_size
        self.kv_pages = torch.zeros(max(1, len(self.attn_layers)), num_pages, 2, self.hkv, page_size, self.d,
                                    dtype=self.kv_dtype, device=self.device)

    def _kv_layer(self, li: int) -> int:
        return self._kv_of[li]

    def kv_bytes_per_token(self) -> int:
        return 2 * self.hkv * self.d * max(1, len(self.attn_layers)) * (2 if self.kv_dtype != torch.float32 else 4)

    def move_tokens(self, moves: torch.Tensor) -> None:
        if moves.numel():
            raise NotImplementedError("a recurrent state cannot drop rejected draft tokens")

    def _grow_state(self) -> None:
        """Add slots: 16 at first, then doubling, up to ``STATE_SLOTS``."""
        n = max(1, len(self.linear_layers))
        add = FIRST_SLOTS if self.capacity == 0 else min(self.capacity, STATE_SLOTS - self.capacity)
        conv = torch.zeros(n, add, self.conv_dim, self.kernel - 1, dtype=torch.float32, device=self.device)
        rec = torch.zeros(n, add, self.nv, self.dk, self.dv, dtype=torch.float32, device=self.device)
        self.conv_state = conv if self.conv_state is None else torch.cat([self.conv_state, conv], dim=1)
        self.rec_state = rec if self.rec_state is None else torch.cat([self.rec_state, rec], dim=1)
        self.free_slots.extend(range(self.capacity + add - 1, self.capacity - 1, -1))
        self.capacity += add

    def _ensure_state(self) -> None:
        if self.rec_state is None:
            self._grow_state()

    def _slot(self, seq_id: int, start_pos: int) -> int:
        slot = self.slot_of.pop(seq_id, None)
        if slot is None:
            if start_pos != 0:
                raise RuntimeError(f"sequence {seq_id} continues at position {start_pos} without a recurrent "
                                   "state (forked or reused sequences are not supported for hybrid models)")
            if not self.free_slots and self.capacity < STATE_SLOTS:
                self._grow_state()
            if not self.free_slots:
                _, slot = self.slot_of.popitem(last=False)
            else:
                slot = self.free_slots.pop()
        if start_pos == 0:
            self.conv_state[:, slot] = 0
            self.rec_state[:, slot] = 0
        self.slot_of[seq_id] = slot
        return slot

    def _fork_state(self, parent: int, child: int) -> None:
        """Parallel samples: the child gets a slot holding a copy of the state its parent reached."""
        src = self.slot_of.pop(parent, None)
        if src is None:
            return
        self.slot_of[parent] = src  # most recently used: taking a slot for the child must not evict it
        dst = self._slot(child, 0)
        self.conv_state[:, dst] = self.conv_state[:, src]
        self.rec_state[:, dst] = self.rec_state[:, src]

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, b: BatchInfo) -> torch.Tensor:
        self._ensure_state()
        for parent, child in np.asarray(getattr(b, "seq_forks", ())).reshape(-1, 2).tolist():
            self._fork_state(int(parent), int(child))
        qi = np.asarray(b.q_indptr)
        ids = [int(s) for s in np.asarray(b.seq_ids).tolist()]
        pos0 = np.asarray(b.start_positions)
        live = [i for i in range(len(ids)) if qi[i + 1] > qi[i]]
        slots = [self._slot(ids[i], int(pos0[i])) for i in live]
        lens = [int(qi[i + 1] - qi[i]) for i in live]
        starts = [int(qi[i]) for i in live]
        self._ctx = {"slots": torch.as_tensor(slots, dtype=torch.long, device=x.device), "lens": lens,
                     "starts": starts, "decode": all(n == 1 for n in lens) and len(live) > 0,
                     "rows": torch.as_tensor(starts, dtype=torch.long, device=x.device)}
        return super().forward(x, b)

    def _attention(self, li: int, h: torch.Tensor, b: BatchInfo) -> torch.Tensor:
        if li in self._lin_of:
            return self._gated_delta_net(li, h)
        pre = f"model.layers.{li}.self_attn."
        qkv = ops.linear(h, self.p.linears[pre + "qkv_proj"])
        gate = ops.linear(h, self.p.linears[pre + "gate_proj"])
        ctx = self._attention_core(li, qkv, b)
        ctx = (ctx.float() * torch.sigmoid(gate.float())).to(h.dtype)
        return ops.linear(ctx, self.p.linears[pre + "o_proj"])

    def _own_gdn_params(self, li: int) -> dict:
        """This rank's part of the unsharded small parameters of a gated delta-rule layer."""
        got = self._gdn_params.get(li)
        if got is None:
            pre = f"model.layers.{li}.linear_attn."
            tp = self.p.tensors
            ba, conv, a_log, dt = (tp[pre + "in_proj_ba.weight"], tp[pre + "conv1d.weight"], tp[pre + "A_log"],
                                   tp[pre + "dt_bias"])
            if self.tp > 1:
                r, nv, kd, vd = self.rank, self.nv, self.key_dim, self.value_dim
                kd_all, vd_all = kd * self.tp, vd * self.tp
                v0 = slice(r * nv, (r + 1) * nv)
                ba = torch.cat([ba[v0], ba[self.nv_all + r * nv: self.nv_all + (r + 1) * nv]]).contiguous()
                conv = torch.cat([conv[r * kd:(r + 1) * kd], conv[kd_all + r * kd: kd_all + (r + 1) * kd],
                                  conv[2 * kd_all + r * vd: 2 * kd_all + (r + 1) * vd]]).contiguous()
                a_log, dt = a_log[v0].contiguous(), dt[v0].contiguous()
            got = self._gdn_params[li] = {"ba": ba, "conv": conv, "A_log": a_log, "dt_bias": dt}
        return got

    def _gated_delta_net(self, li: int, h: torch.Tensor) -> torch.Tensor:
        pre = f"model.layers.{li}.linear_attn."
        t_all = h.shape[0]
        tp = self.p.tensors
        own = self._own_gdn_params(li)
        ctx = self._ctx
        layer = self._lin_of[li]
        proj = ops.linear(h, self.p.linears[pre + "in_proj_qkvz"]).float()
        mixed, z = proj[:, : self.conv_dim], proj[:, self.conv_dim:]
        ba = h.float() @ own["ba"].float().t()
        beta = torch.sigmoid(ba[:, : self.nv])
        g = -own["A_log"].exp() * F.softplus(ba[:, self.nv:] + own["dt_bias"])
        w = own["conv"]                                                  # [conv_dim, K]
        slots = ctx["slots"]
        conv_all = self.conv_state[layer]
        rec_all = self.rec_state[layer]
        out = torch.empty(t_all, self.nv, self.dv, dtype=torch.float32, device=h.device)
        rep = self.nv // self.nk

        def heads(conv_out: torch.Tensor):
            """Convolved rows [N, conv_dim] -> normalised q, k [N, nv, dk] and v [N, nv, dv]."""
            q, k, v = torch.split(F.silu(conv_out), [self.key_dim, self.key_dim, self.value_dim], dim=-1)
            q = q.reshape(-1, self.nk, self.dk)
            k = k.reshape(-1, self.nk, self.dk)
            q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * (self.dk ** -0.5)
            k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            if rep > 1:
                q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
            return q, k, v.reshape(-1, self.nv, self.dv)

        if ctx["decode"]:
            # one token per sequence: one batched window product and one batched state update
            rows = ctx["rows"]
            window = torch.cat([conv_all[slots], mixed[rows].unsqueeze(-1)], dim=-1)   # [B, conv_dim, K]
            conv_all[slots] = window[:, :, 1:]
            q, k, v = heads((window * w.unsqueeze(0)).sum(-1))
            if not _gdn_step_kernel(rec_all, slots, q, k, v, g[rows], beta[rows], out, rows):
                state = rec_all[slots]
                out[rows] = gated_delta_step(state, q, k, v, g[rows], beta[rows])
                rec_all[slots] = state
        else:
            for j, (start, n) in enumerate(zip(ctx["starts"], ctx["lens"])):
                slot = slots[j]
                seq = torch.cat([conv_all[slot], mixed[start:start + n].t()], dim=-1)   # [conv_dim, K - 1 + n]
                conv_all[slot] = seq[:, -(self.kernel - 1):]
                conv = F.conv1d(seq.unsqueeze(0), w.unsqueeze(1), groups=self.conv_dim)[0].t()  # [n, conv_dim]
                q, k, v = heads(conv)
                state = rec_all[slot].clone()
                out[start:start + n] = gated_delta_chunk(state, q, k, v, g[start:start + n], beta[start:start + n])
                rec_all[slot] = state
        # gated RMS norm over every value head, then the output projection
        o = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps)
        o = o * tp[pre + "norm.weight"].view(1, 1, -1) * F.silu(z.reshape(t_all, self.nv, self.dv))
        return ops.linear(o.reshape(t_all, self.value_dim).to(h.dtype), self.p.linears[pre + "out_proj"])
