"""RWKV-5 ("Eagle") and RWKV-6 ("Finch"): recurrent models whose per-sequence state replaces the KV cache.

Reference: ``python/mlc_llm/model/rwkv5/rwkv5_model.py`` (time-mix block with a per-head matrix state
updated by the ``wkv5`` recurrence ``:64-123``, channel-mix block ``:150-175``, token shift against the
previous token ``:127-146``, LayerNorm before the first block, halving of the activations every
``rescale_every`` blocks) and ``python/mlc_llm/nn/rnn_state.py`` (one state slot per sequence and layer:
the last input of each of the two blocks plus the matrix state).

The engine drives this model like any other: tokens arrive per sequence, possibly in chunks, and the
sequence id selects the state.  What a recurrent state cannot do is roll back or be shared: speculative
decoding, jump-forward roll-back, prefix reuse and forked parallel samples are not available for this
family (the runtime switches the prefix cache off).

The recurrence itself runs as one pass over the tokens of each sequence in fp32:

    out_t[i] = sum_k r_t[k] * (u[k] * k_t[k] * v_t[i] + S[i, k])
    S[i, k]  = S[i, k] * w[k] + k_t[k] * v_t[i]

with ``w = exp(-exp(time_decay))`` and ``u = time_faaaa`` per head.  RWKV-6
(``python/mlc_llm/model/rwkv6/rwkv6_model.py``) keeps the recurrence and makes two things depend on the
token: the token-shift mixing weights get low-rank corrections, and the decay ``w`` is computed per token.
"""

from __future__ import annotations

import collections
from typing import Dict, Optional

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from .transformer import BatchInfo, DecoderModel

STATE_CAP = 4096  # sequences whose state is remembered; the least recently used go first


def wkv5(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor,
         state: torch.Tensor) -> torch.Tensor:
    """One sequence: ``r, k, v [T, N, H]`` fp32, ``u [N, H]``, decay ``w [N, H]`` (RWKV-5) or ``[T, N, H]``
    (RWKV-6, one decay per token), ``state [N, H(value), H(key)]`` updated in place; returns ``[T, N, H]``."""
    t_len = r.shape[0]
    out = torch.empty_like(r)
    for t in range(t_len):
        kv = v[t].unsqueeze(-1) * k[t].unsqueeze(-2)                      # [N, Hv, Hk]
        out[t] = ((u.unsqueeze(-2) * kv + state) * r[t].unsqueeze(-2)).sum(-1)
        wt = w[t] if w.dim() == 3 else w
        state.mul_(wt.unsqueeze(-2)).add_(kv)
    return out


def wkv5_batch(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor,
               kv_states, layer_pos: int, q_indptr: np.ndarray) -> torch.Tensor:
    """All sequences of a step: ``kv_states[i]`` is sequence i's ``[layers, N, H, H]`` fp32 state (row
    ``layer_pos`` is updated in place).  On a GPU with head size 32 / 64 this is one launch of
    ``wkv5_kernel``; otherwise the per-sequence loop above."""
    t_all, n, hs = r.shape
    out = torch.empty(t_all, n, hs, dtype=torch.float32, device=r.device)
    if r.is_cuda and hs in (32, 64) and len(kv_states) <= 65535:
        import ctypes  # pylint: disable=import-outside-toplevel

        from ..ops._lib import check, lib, ptr, stream_ptr  # pylint: disable=import-outside-toplevel

        for st in kv_states:
            assert st.is_contiguous() and st.dtype == torch.float32
        base = torch.tensor([st.data_ptr() for st in kv_states], dtype=torch.int64).to(r.device)
        qi = torch.from_numpy(np.ascontiguousarray(q_indptr, dtype=np.int32)).to(r.device)
        layer_offset = layer_pos * n * hs * hs
        rc = lib().mlcb_wkv5(ptr(r.contiguous()), ptr(k.contiguous()), ptr(v.contiguous()), ptr(w.contiguous()),
                             ptr(u.contiguous()), ptr(base), ctypes.c_longlong(layer_offset), ptr(qi), ptr(out),
                             ctypes.c_int(len(kv_states)), ctypes.c_int(n), ctypes.c_int(hs), ctypes.c_int(t_all),
                             ctypes.c_int(1 if w.dim() == 3 else 0), stream_ptr())
        check(rc, "mlcb_wkv5")
        return out
    for i, st in enumerate(kv_states):
        s, e = int(q_indptr[i]), int(q_indptr[i + 1])
        if e > s:
            out[s:e] = wkv5(r[s:e], k[s:e], v[s:e], w[s:e] if w.dim() == 3 else w, u, st[layer_pos])
    return out


class RwkvModel(DecoderModel):
    """RWKV-5 behind the decoder-model interface of the executor."""

    stateful = True  # per-sequence recurrent state: no paged KV, no CUDA-graph replay of the forward

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        c = self.cfg
        # tensor parallelism: a rank keeps `heads` whole heads of the time-mix block (their projections, decay,
        # bonus, group norm and matrix state) and a slice of the channel-mix width; token-shift vectors and the
        # residual stream are whole on every rank (reference: rwkv6_model.py shard strategies)
        total = c.hidden_size // c.head_dim
        if total % self.tp:
            raise ValueError(f"{total} heads cannot be split over {self.tp} ranks")
        self.heads = total // self.tp
        rank = self.comm.tp_rank if (self.comm is not None and self.tp > 1) else 0
        self._lo, self._hi = rank * self.heads * c.head_dim, (rank + 1) * self.heads * c.head_dim
        self.states: "collections.OrderedDict[int, Dict[str, torch.Tensor]]" = collections.OrderedDict()

    # ------------------------------------------------------------------ state
    def create_kv_cache(self, num_pages: int, page_size: int = 16) -> None:
        self.page = page_size
        self.kv_pages = torch.zeros(0, dtype=self.kv_dtype, device=self.device)  # nothing is paged

    def copy_pages(self, pairs: torch.Tensor) -> None:
        return

    def move_tokens(self, moves: torch.Tensor) -> None:
        if moves.numel():
            raise NotImplementedError("a recurrent state cannot drop rejected draft tokens")

    def state_bytes_per_sequence(self) -> int:
        """What one sequence's recurrent state occupies (two shift vectors and one matrix state per head and
        layer): the engine's capacity inference sizes the batch by it."""
        c, n = self.cfg, len(self.layers)
        es = torch.empty((), dtype=self.dtype).element_size()
        return n * (2 * c.hidden_size * es + self.heads * c.head_dim * c.head_dim * 4)

    def _fresh_state(self) -> Dict[str, torch.Tensor]:
        c, n = self.cfg, len(self.layers)
        return {"att_x": torch.zeros(n, c.hidden_size, dtype=self.dtype, device=self.device),
                "ffn_x": torch.zeros(n, c.hidden_size, dtype=self.dtype, device=self.device),
                "kv": torch.zeros(n, self.heads, c.head_dim, c.head_dim, dtype=torch.float32, device=self.device)}

    def _state_of(self, seq_id: int, start_pos: int) -> Dict[str, torch.Tensor]:
        st = self.states.pop(seq_id, None)
        if st is None or start_pos == 0:
            if start_pos != 0:
                raise RuntimeError(f"sequence {seq_id} continues at position {start_pos} without a recurrent "
                                   "state (forked or reused sequences are not supported for RNN models)")
            st = self._fresh_state()
        self.states[seq_id] = st
        while len(self.states) > STATE_CAP:
            self.states.popitem(last=False)
        return st

    # ------------------------------------------------------------------ forward
    def embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.p.tensors["model.embeddings.weight"][token_ids.long()].to(self.dtype)

    def _own(self, t: torch.Tensor) -> torch.Tensor:
        """This rank's heads of a per-channel parameter whose last dimension(s) span all heads."""
        if self.tp == 1:
            return t
        c = self.cfg
        if t.shape[-1] == c.hidden_size:
            return t[..., self._lo:self._hi]
        return t.reshape(*t.shape[:-2], c.hidden_size)[..., self._lo:self._hi].reshape(
            *t.shape[:-2], self.heads, c.head_dim)

    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return F.layer_norm(x.float(), (x.shape[-1],), self.p.tensors[name + ".weight"].float(),
                            self.p.tensors[name + ".bias"].float(), self.cfg.rms_norm_eps).to(x.dtype)

    @staticmethod
    def _shift(x: torch.Tensor, prev: torch.Tensor, starts: np.ndarray, firsts: torch.Tensor) -> torch.Tensor:
        """Row t gets row t - 1; the first row of every sequence gets that sequence's stored last input."""
        sx = torch.roll(x, 1, dims=0)
        sx[firsts] = prev
        return sx

    def forward(self, x: torch.Tensor, b: BatchInfo) -> torch.Tensor:
        c = self.cfg
        qi = np.asarray(b.q_indptr)
        ids = [int(s) for s in np.asarray(b.seq_ids).tolist()]
        pos0 = np.asarray(b.start_positions)
        live = [i for i in range(len(ids)) if qi[i + 1] > qi[i]]
        for parent, child in np.asarray(getattr(b, "seq_forks", ())).reshape(-1, 2).tolist():
            # parallel samples: the child continues from a copy of the state its parent reached
            st = self.states.get(int(parent))
            if st is not None:
                self.states[int(child)] = {k: v.clone() for k, v in st.items()}
        states = {i: self._state_of(ids[i], int(pos0[i])) for i in live}
        firsts = torch.as_tensor([int(qi[i]) for i in live], dtype=torch.long, device=x.device)
        lasts = torch.as_tensor([int(qi[i + 1]) - 1 for i in live], dtype=torch.long, device=x.device)
        hs, n = c.head_dim, self.heads
        t_all = x.shape[0]
        v6 = int(c.extra.get("rwkv", 5)) == 6
        # chunk boundaries of the sequences that have tokens in this step (they are contiguous in x)
        live_indptr = np.asarray([int(qi[i]) for i in live] + [int(qi[live[-1] + 1]) if live else 0], dtype=np.int32)
        for pos, li in enumerate(self.layers):
            pre = f"model.blocks.{li}."
            if li == 0:
                x = self._ln(x, pre + "pre_ln")
            # ---- time mix
            h = self._ln(x, pre + "ln1")
            prev = torch.stack([states[i]["att_x"][pos] for i in live])
            sx = self._shift(h, prev, qi, firsts)
            a = pre + "attention."
            if v6:
                # data-dependent interpolation: five low-rank corrections of the mixing weights, and a
                # per-token decay (reference: python/mlc_llm/model/rwkv6/rwkv6_model.py:236-272)
                tp = self.p.tensors
                dx = sx - h
                xxx = torch.tanh((h + dx * tp[a + "time_maa_x"]).float() @ tp[a + "time_maa_w1"].float())
                xxx = xxx.view(t_all, 5, -1).transpose(0, 1)                       # [5, T, D]
                m5 = torch.bmm(xxx, tp[a + "time_maa_w2"].float()).to(h.dtype)      # [5, T, hidden]
                mixed = lambda j, name: h + dx * (tp[a + name] + m5[j])
                xw, xk, xv, xr, xg = (mixed(0, "time_maa_w"), mixed(1, "time_maa_k"), mixed(2, "time_maa_v"),
                                      mixed(3, "time_maa_r"), mixed(4, "time_maa_g"))
                dec = self._own(tp[a + "time_decay"]).float().view(1, n, hs) + (
                    torch.tanh(xw.float() @ tp[a + "time_decay_w1"].float()) @ self._own(tp[a + "time_decay_w2"]).float()
                ).view(t_all, n, hs)
                w = torch.exp(-torch.exp(dec)).contiguous()
            else:
                mix = lambda name: h * self.p.tensors[a + name] + sx * (1.0 - self.p.tensors[a + name])
                xr, xk, xv, xg = (mix("time_mix_receptance"), mix("time_mix_key"), mix("time_mix_value"),
                                  mix("time_mix_gate"))
                w = self._own(self.p.tensors[a + "time_decay"]).float()
            r = ops.linear(xr, self.p.linears[a + "receptance"]).float().view(t_all, n, hs)
            k = ops.linear(xk, self.p.linears[a + "key"]).float().view(t_all, n, hs)
            v = ops.linear(xv, self.p.linears[a + "value"]).float().view(t_all, n, hs)
            g = F.silu(ops.linear(xg, self.p.linears[a + "gate"]).float())
            u = self._own(self.p.tensors[a + "time_faaaa"]).float()
            out = wkv5_batch(r, k, v, w, u, [states[i]["kv"] for i in live], pos, live_indptr)
            newest = h.index_select(0, lasts)
            for j, i in enumerate(live):
                states[i]["att_x"][pos] = newest[j]
            out = F.group_norm(out.view(t_all, n * hs), n, self._own(self.p.tensors[a + "ln_x.weight"]).float(),
                               self._own(self.p.tensors[a + "ln_x.bias"]).float(), eps=1e-5)
            x = x + self._reduce(ops.linear((out * g).to(self.dtype), self.p.linears[a + "output"]))
            # ---- channel mix
            h = self._ln(x, pre + "ln2")
            prev = torch.stack([states[i]["ffn_x"][pos] for i in live])
            sx = self._shift(h, prev, qi, firsts)
            f = pre + "feed_forward."
            if v6:
                xk = h + (sx - h) * self.p.tensors[f + "time_maa_k"]
                xr = h + (sx - h) * self.p.tensors[f + "time_maa_r"]
            else:
                xk = h * self.p.tensors[f + "time_mix_key"] + sx * (1.0 - self.p.tensors[f + "time_mix_key"])
                xr = h * self.p.tensors[f + "time_mix_receptance"] + sx * (1.0 - self.p.tensors[f + "time_mix_receptance"])
            newest = h.index_select(0, lasts)
            for j, i in enumerate(live):
                states[i]["ffn_x"][pos] = newest[j]
            rr = torch.sigmoid(ops.linear(xr, self.p.linears[f + "receptance"]).float())
            kk = torch.square(torch.relu(ops.linear(xk, self.p.linears[f + "key"]).float())).to(self.dtype)
            x = x + (rr * self._reduce(ops.linear(kk, self.p.linears[f + "value"])).float()).to(self.dtype)
            rescale = int(c.extra.get("rescale_every", 0))
            if rescale > 0 and (li + 1) % rescale == 0:
                x = x / 2.0
        self._final_normed = None
        return x

    def logits(self, hidden: torch.Tensor, rows: Optional[torch.Tensor]) -> torch.Tensor:
        src = hidden if rows is None else hidden.index_select(0, rows.long())
        h = self._ln(src, "model.ln_out")
        return ops.linear(h, self.p.linears["head"], out_dtype=torch.float32)
