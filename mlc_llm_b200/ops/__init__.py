"""Operator front-end: every function takes torch tensors and runs the hand-written sm_100a kernel
when the tensors live on a GPU, or the fp32 PyTorch restatement (``ops.reference``) on CPU.

There is no silent fallback on a GPU: a shape a kernel does not take raises ``KernelError``.
"""

from __future__ import annotations

import ctypes
import dataclasses
import os
from typing import Optional

import torch

from .. import quantization as Q
from . import reference as ref
from ._lib import DTYPE_CODE, KernelError, check, check_status, lib, ptr, status_word, stream_ptr

c_int = ctypes.c_int
c_float = ctypes.c_float
c_ll = ctypes.c_longlong


# --------------------------------------------------------------------------- linear
@dataclasses.dataclass
class LinearWeight:
    """A linear layer's parameters in their run-time layout.

    kind ``dense``: ``w [N, K]``.  kind ``q4``: ``w`` is packed int4 ``[N, K/8]`` int32 (artifact
    nibble order on CPU, device order on GPU -- see ``quantization.to_device_layout_q4``) and
    ``scale [N, K/32]``; on a GPU the tensor-core GEMM reads a second, tile-record form of the same
    data (:meth:`q4_tiles`, ``quantization.to_tiled_q4``), the one-to-four-token GEMV the row-major
    one.  kind ``fp8_block``: ``w [N, K]`` e4m3, ``scale [N/128, K/128]`` fp32.
    kind ``fp8_tensor``: fp8 ``w`` with a scalar ``scale``.
    """

    kind: str
    w: torch.Tensor
    scale: Optional[torch.Tensor] = None
    bias: Optional[torch.Tensor] = None
    quant: Optional[Q.Quantization] = None
    out_features: int = 0
    in_features: int = 0
    device_layout: bool = False
    # dense fp16/bf16 copy used by kernels that do not take the packed form (built lazily)
    _dense: Optional[torch.Tensor] = None
    _block_scale: Optional[torch.Tensor] = None
    # int4 tile records for the tensor-core GEMM (GPU only, built when the weight moves to the GPU)
    _tiles: Optional[torch.Tensor] = None

    def q4_tiles(self) -> torch.Tensor:
        if self._tiles is None:
            assert self.kind == "q4" and self.device_layout and self.w.is_cuda
            self._tiles = Q.to_tiled_q4(self.w, self.scale)
        return self._tiles

    def q4_tileable(self, k: int) -> bool:
        """The tensor-core int4 path needs 4-bit groups of 32, K a multiple of 64 and, for stacked
        expert slabs, slabs of whole 128-row blocks."""
        return (self.kind == "q4" and self.quant is not None and self.quant.bits == 4
                and self.quant.group_size == 32 and k % 64 == 0 and self.scale is not None
                and self.scale.dtype in (torch.float16, torch.bfloat16)
                and (self.w.dim() == 2 or self.w.shape[-2] % 128 == 0))

    def to(self, device) -> "LinearWeight":
        dev = torch.device(device)
        w, dl = self.w, self.device_layout
        if self.kind == "q4" and self.quant is not None and self.quant.bits == 4:
            if dev.type == "cuda" and not dl:
                w, dl = Q.to_device_layout_q4(w), True
            elif dev.type == "cpu" and dl:
                w, dl = Q.from_device_layout_q4(w.cpu()), False
        out = LinearWeight(self.kind, w.to(dev), None if self.scale is None else self.scale.to(dev),
                           None if self.bias is None else self.bias.to(dev), self.quant,
                           self.out_features, self.in_features, dl)
        if dev.type == "cuda" and dl and out.q4_tileable(w.shape[-1] * 8):
            out.q4_tiles()
        return out

    def block_scale(self) -> torch.Tensor:
        """fp32 scales ``[ceil(N/128), ceil(K/128)]`` of an fp8 weight as the block-scaled GEMM kernels read
        them. A per-tensor scale is one value repeated, so per-tensor fp8 checkpoints run on the same
        kernels (reference: the per-tensor mode dequantises inside its matmul,
        ``python/mlc_llm/quantization/per_tensor_quantization.py``)."""
        if self.kind == "fp8_block":
            if self.scale.dtype != torch.float32 or not self.scale.is_contiguous():
                self.scale = self.scale.float().contiguous()
            return self.scale
        if self.kind != "fp8_tensor":
            raise ValueError(self.kind)
        if self._block_scale is None:
            n, k = self.w.shape[-2], self.w.shape[-1]
            self._block_scale = self.scale.float().reshape(-1)[:1].expand(
                (n + 127) // 128 * ((k + 127) // 128)).reshape((n + 127) // 128, (k + 127) // 128).contiguous()
        return self._block_scale

    def dense(self, dtype: torch.dtype) -> torch.Tensor:
        """Materialise the full-precision weight (used by oracles and by cold paths)."""
        if self.kind == "dense":
            return self.w.to(dtype)
        if self._dense is None or self._dense.dtype != dtype:
            if self.kind == "q4":
                qw = Q.from_device_layout_q4(self.w) if self.device_layout else self.w
                self._dense = Q.group_dequantize(qw, self.scale, self.quant, k=self.in_features,
                                                 out_dtype=dtype)
            elif self.kind == "fp8_block":
                self._dense = Q.fp8_block_dequantize(self.w, self.scale, out_dtype=dtype)
            elif self.kind == "fp8_tensor":
                self._dense = (self.w.float() * self.scale.float()).to(dtype)
            else:
                raise ValueError(self.kind)
        return self._dense


def dense_weight(w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> LinearWeight:
    return LinearWeight("dense", w, None, bias, None, w.shape[0], w.shape[1])


# grouped (mixture-of-experts) products with at most this many rows take the GEMV form
_MOE_GEMV_MAX_ROWS = int(os.environ.get("MLCB_MOE_GEMV_MAX_ROWS", "8"))
_WARNED_DENSE = set()


def _warn_dense_fallback(lw: "LinearWeight", k: int) -> None:
    """Quantisation layouts without a kernel of their own (3-bit groups, K-major ``*_0`` packing, fp32 scales,
    K not a multiple of 64, ...) run on a dequantised 16-bit copy of the weight: correct, but the memory saving
    is gone. Said once per layout, not silently."""
    name = getattr(lw.quant, "name", None) or lw.kind
    key = (name, k % 64 == 0)
    if key in _WARNED_DENSE:
        return
    _WARNED_DENSE.add(key)
    import logging  # pylint: disable=import-outside-toplevel

    logging.getLogger("mlc_llm_b200").warning(
        "quantization %s (K = %d) has no packed-weight kernel: its linear layers run on a dequantised 16-bit copy "
        "of the weights (full 16-bit memory footprint)", name, k)


_GEMM_SCRATCH = {}
GEMM_WORKSPACE_BYTES = 32 << 20
GEMM_COUNTERS = 4096


def _gemm_scratch(device: torch.device):
    """Split-K scratch of the GEMM kernel: fp32 partial sums plus per-tile arrival counters
    (zero between launches). One per device; launches on one device are stream-ordered."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    sc = _GEMM_SCRATCH.get(key)
    if sc is None:
        ws = torch.empty(GEMM_WORKSPACE_BYTES // 4, dtype=torch.float32, device=device)
        cnt = torch.zeros(GEMM_COUNTERS, dtype=torch.int32, device=device)
        sc = (ws, cnt)
        _GEMM_SCRATCH[key] = sc
    return (ptr(sc[0]), c_ll(GEMM_WORKSPACE_BYTES), ptr(sc[1]), c_int(GEMM_COUNTERS))


_LINEAR_OBSERVER = None
_GEMV_Q4 = os.environ.get("MLCB_GEMV_Q4", "1") != "0"
_LOWM_Q4 = os.environ.get("MLCB_LOWM_Q4", "0") != "0"


def set_linear_observer(fn) -> None:
    """Install ``fn(weight, activations [M, K])`` to be called before every :func:`linear` (None removes
    it).  Used by calibration to record activation statistics; not meant for the serving path."""
    global _LINEAR_OBSERVER  # pylint: disable=global-statement
    _LINEAR_OBSERVER = fn


def linear(x: torch.Tensor, lw: LinearWeight, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``y = x @ W^T (+ bias)`` for ``x [..., K]``."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if _LINEAR_OBSERVER is not None and x2.shape[0] > 0:
        _LINEAR_OBSERVER(lw, x2)
    od = out_dtype or x.dtype
    if not x.is_cuda:
        w = lw.dense(torch.float32)
        y = ref.linear_dense(x2, w, lw.bias, od)
        return y.reshape(*lead, -1)
    m, k = x2.shape
    n = lw.out_features or lw.w.shape[0]
    if x2.dtype not in (torch.float16, torch.bfloat16):
        raise KernelError(f"linear: unsupported activation dtype {x2.dtype}")
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    y = torch.empty(m, n, dtype=od, device=x.device)
    if m == 0:
        return y.reshape(*lead, n)
    ab = DTYPE_CODE[x2.dtype]
    if lw.q4_tileable(k) and x2.dtype == lw.scale.dtype:
        assert lw.device_layout
        if m <= 4 and od in (torch.float16, torch.float32) and _GEMV_Q4 and x2.dtype == torch.float16:
            # one to four tokens: the memory-bound CUDA-core kernel beats the tensor-core one, whose
            # dequantise stage is sized for wide token tiles
            rc = lib().mlcb_gemv_q4(ptr(x2), ptr(lw.w), ptr(lw.scale), ptr(lw.bias), ptr(y), c_int(m), c_int(n),
                                    c_int(k), c_int(x2.stride(0)), c_int(n), c_int(DTYPE_CODE[od]), stream_ptr())
            if rc == 0:
                return y.reshape(*lead, n)
            if rc > 0:
                check(rc, f"mlcb_gemv_q4(M={m},N={n},K={k})")
        elif m <= 16 and od in (torch.float16, torch.float32) and _LOWM_Q4 and x2.dtype == torch.float16:
            # five to sixteen tokens: nibbles expanded in registers into warp-level MMA fragments
            rc = lib().mlcb_gemm_q4_lowm(ptr(x2), ptr(lw.w), ptr(lw.scale), ptr(lw.bias), ptr(y), c_int(m), c_int(n),
                                         c_int(k), c_int(x2.stride(0)), c_int(n), c_int(DTYPE_CODE[od]), stream_ptr())
            if rc == 0:
                return y.reshape(*lead, n)
            if rc > 0:
                check(rc, f"mlcb_gemm_q4_lowm(M={m},N={n},K={k})")
        tiles = lw.q4_tiles()
        rc = lib().mlcb_gemm(ptr(x2), ptr(tiles), ptr(tiles), ptr(lw.bias), ptr(y), c_int(m),
                             c_int(n), c_int(k), c_int(x2.stride(0)), c_int(n), c_int(ab),
                             c_int(DTYPE_CODE[od]), ptr(status_word(x.device)), *_gemm_scratch(x.device),
                             stream_ptr())
    elif lw.kind in ("fp8_block", "fp8_tensor") and k % 64 == 0 and lw.w.dtype == torch.float8_e4m3fn \
            and lw.w.dim() == 2:
        from .fp8 import linear_fp8_block  # pylint: disable=import-outside-toplevel

        return linear_fp8_block(x2, lw, od).reshape(*lead, n)
    else:
        if lw.kind != "dense" and lw._dense is None:
            _warn_dense_fallback(lw, k)
        w = lw.dense(x2.dtype)
        rc = lib().mlcb_gemm(ptr(x2), ptr(w), ptr(None), ptr(lw.bias), ptr(y), c_int(m), c_int(n),
                             c_int(k), c_int(x2.stride(0)), c_int(n), c_int(ab),
                             c_int(DTYPE_CODE[od]), ptr(status_word(x.device)), *_gemm_scratch(x.device),
                             stream_ptr())
    check(rc, f"mlcb_gemm(M={m},N={n},K={k},{lw.kind})")
    return y.reshape(*lead, n)


# --------------------------------------------------------------------------- norms / activations
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, w_offset: float = 0.0) -> torch.Tensor:
    if not x.is_cuda:
        return ref.rmsnorm(x, w, eps, w_offset)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    out = torch.empty_like(x2)
    rc = lib().mlcb_rmsnorm(ptr(x2), ptr(None), ptr(w), ptr(out), c_int(x2.shape[0]),
                            c_int(x2.shape[1]), c_float(eps), c_float(w_offset),
                            c_int(DTYPE_CODE[x.dtype]), stream_ptr())
    check(rc, "mlcb_rmsnorm")
    return out.reshape(x.shape)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float,
                w_offset: float = 0.0) -> torch.Tensor:
    """``residual += x`` in place; returns ``rmsnorm(residual)``. Both ``[T, H]`` contiguous."""
    if not x.is_cuda:
        return ref.add_rmsnorm(x, residual, w, eps, w_offset)
    assert x.is_contiguous() and residual.is_contiguous()
    out = torch.empty_like(x)
    rc = lib().mlcb_rmsnorm(ptr(x), ptr(residual), ptr(w), ptr(out), c_int(x.shape[0]),
                            c_int(x.shape[1]), c_float(eps), c_float(w_offset),
                            c_int(DTYPE_CODE[x.dtype]), stream_ptr())
    check(rc, "mlcb_rmsnorm(add)")
    return out


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float,
              residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm over the last dimension; with ``residual``: ``residual += x`` in place first and the norm
    is taken of the sum (reference: ``nn.LayerNorm`` in e.g. ``python/mlc_llm/model/gpt2/gpt2_model.py``)."""
    h = x.shape[-1]
    ok = (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and h % 8 == 0 and h <= 12000
          and w.dtype == x.dtype and (b is None or b.dtype == x.dtype))
    if not ok:
        if residual is not None:
            residual.add_(x)
            x = residual
        return ref.layernorm(x, w, b, eps)
    x2 = x.reshape(-1, h)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if residual is not None:
        assert residual.is_contiguous() and residual.shape == x.shape
    out = torch.empty_like(x2)
    rc = lib().mlcb_layernorm(ptr(x2), ptr(residual), ptr(w.contiguous()), ptr(None if b is None else b.contiguous()),
                              ptr(out), c_int(x2.shape[0]), c_int(h), c_float(eps), c_int(DTYPE_CODE[x.dtype]),
                              stream_ptr())
    check(rc, "mlcb_layernorm")
    return out.reshape(x.shape)


_ACT_CODE = {"silu": 0, "gelu_tanh": 1, "gelu": 2, "relu2": 3, "quick_gelu": 4}


def activation(x: torch.Tensor, act: str) -> torch.Tensor:
    """Elementwise ``silu`` / ``gelu`` (erf) / ``gelu_tanh`` / ``relu2`` (squared ReLU) / ``quick_gelu``
    (``x * sigmoid(1.702 x)``, CLIP)."""
    if not (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and x.numel() % 8 == 0 and x.is_contiguous()):
        xf = x.float()
        if act == "silu":
            y = torch.nn.functional.silu(xf)
        elif act == "gelu":
            y = torch.nn.functional.gelu(xf)
        elif act == "gelu_tanh":
            y = torch.nn.functional.gelu(xf, approximate="tanh")
        elif act == "relu2":
            y = torch.relu(xf) ** 2
        elif act == "quick_gelu":
            y = xf * torch.sigmoid(1.702 * xf)
        else:
            raise ValueError(act)
        return y.to(x.dtype)
    out = torch.empty_like(x)
    rc = lib().mlcb_act(ptr(x), ptr(out), ctypes.c_longlong(x.numel()), c_int(_ACT_CODE[act]),
                        c_int(DTYPE_CODE[x.dtype]), stream_ptr())
    check(rc, "mlcb_act")
    return out


def act_mul(x: torch.Tensor, act: str = "silu", live_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(gate) * up`` of ``[.., 2 * I]`` rows. ``live_rows`` (int32 device scalar): only that many leading rows
    are computed, the rest of the output is left as allocated."""
    if not x.is_cuda:
        return ref.act_mul(x, act)
    assert x.is_contiguous()
    inter = x.shape[-1] // 2
    out = torch.empty(*x.shape[:-1], inter, dtype=x.dtype, device=x.device)
    tokens = x.numel() // x.shape[-1]
    rc = lib().mlcb_act_mul(ptr(x), ptr(out), c_int(tokens), c_int(inter),
                            c_int(0 if act == "silu" else 1), c_int(DTYPE_CODE[x.dtype]), stream_ptr(),
                            ptr(live_rows))
    check(rc, "mlcb_act_mul")
    return out


def embed(ids: torch.Tensor, table, hidden: int, dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    """Embedding lookup. ``table`` is a dense tensor ``[V, H]`` or a q4 ``LinearWeight`` in the
    artifact nibble order (the embedding table is never re-laid-out)."""
    if isinstance(table, LinearWeight) and table.kind == "q4":
        if not ids.is_cuda:
            rows = Q.group_dequantize(table.w[ids.long()], table.scale[ids.long()], table.quant,
                                      k=hidden, out_dtype=dtype)
            return rows * scale if scale != 1.0 else rows
        out = torch.empty(ids.shape[0], hidden, dtype=torch.float16, device=ids.device)
        rc = lib().mlcb_embed_q4(ptr(ids), ptr(table.w), ptr(table.scale), ptr(out),
                                 c_int(ids.shape[0]), c_int(hidden), c_int(table.w.shape[0]),
                                 stream_ptr())
        check(rc, "mlcb_embed_q4")
        if scale != 1.0:
            out = out * scale
        return out.to(dtype)
    tbl = table.w if isinstance(table, LinearWeight) else table
    if not ids.is_cuda:
        rows = tbl[ids.long()].to(dtype)
        return rows * scale if scale != 1.0 else rows
    out = torch.empty(ids.shape[0], hidden, dtype=tbl.dtype, device=ids.device)
    rc = lib().mlcb_embed(ptr(ids), ptr(tbl), ptr(out), c_int(ids.shape[0]), c_int(hidden),
                          c_int(tbl.shape[0]), c_float(scale), c_int(DTYPE_CODE[tbl.dtype]),
                          stream_ptr())
    check(rc, "mlcb_embed")
    return out


# --------------------------------------------------------------------------- RoPE + KV append
def rope_append(qkv: torch.Tensor, kv_pages: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor,
                inv_freq: Optional[torch.Tensor], hq: int, hkv: int, d: int, rot_dim: int, page: int,
                attn_factor: float = 1.0) -> None:
    if not qkv.is_cuda:
        ref.rope_append(qkv, kv_pages, pos, slot, inv_freq, hq, hkv, d, rot_dim, page, attn_factor)
        return
    assert qkv.is_contiguous() and kv_pages.is_contiguous()
    if inv_freq is None:
        rot_dim = 0
        inv_freq = torch.zeros(1, dtype=torch.float32, device=qkv.device)
    num_slots = kv_pages.shape[0] * page
    rc = lib().mlcb_rope_append(ptr(qkv), ptr(kv_pages), ptr(pos), ptr(slot), ptr(inv_freq),
                                c_int(qkv.shape[0]), c_int(hq), c_int(hkv), c_int(d), c_int(rot_dim),
                                c_int(page), c_float(attn_factor), c_ll(num_slots),
                                c_int(DTYPE_CODE[qkv.dtype]), ptr(status_word(qkv.device)),
                                stream_ptr())
    check(rc, "mlcb_rope_append")


# --------------------------------------------------------------------------- attention
def paged_attention(q: torch.Tensor, kv_pages: torch.Tensor, q_seq: torch.Tensor,
                    q_kvlen: torch.Tensor, page_indptr: torch.Tensor, page_indices: torch.Tensor,
                    hq: int, hkv: int, d: int, page: int, sm_scale: float,
                    q_kvstart: Optional[torch.Tensor] = None, sink: int = 0,
                    tree_mask: Optional[torch.Tensor] = None, softcap: float = 0.0,
                    return_lse: bool = False, plan=None):
    """``q``: ``[T, hq*d]`` view (row stride may exceed ``hq*d``). Returns ``[T, hq*d]``."""
    t = q.shape[0]
    if not q.is_cuda:
        res = ref.paged_attention(q.reshape(t, hq, d), kv_pages, q_seq, q_kvlen, page_indptr,
                                  page_indices, hq, hkv, d, page, sm_scale, q_kvstart, sink,
                                  tree_mask, softcap, return_lse)
        if return_lse:
            return res[0].reshape(t, hq * d), res[1]
        return res.reshape(t, hq * d)
    out = torch.empty(t, hq * d, dtype=q.dtype, device=q.device)
    lse = torch.empty(t, hq, dtype=torch.float32, device=q.device) if return_lse else None
    if plan is not None and plan.use_tensor_core and d == 128 and page == 16 \
            and q.dtype in (torch.float16, torch.bfloat16):
        from .attention import attention_decode, attention_tcgen05  # pylint: disable=import-outside-toplevel

        if plan.num_dec:
            attention_decode(q, kv_pages, out, lse, plan, hq, hkv, sm_scale, q_kvstart=q_kvstart, sink=sink,
                             tree_mask=tree_mask, softcap=softcap)
        if plan.num_tiles:
            attention_tcgen05(q, kv_pages, out, lse, plan, hq, hkv, sm_scale, q_kvstart=q_kvstart, sink=sink,
                              tree_mask=tree_mask, softcap=softcap)
    else:
        rc = lib().mlcb_attn_simt(ptr(q), ptr(kv_pages), ptr(out), ptr(lse), ptr(q_seq), ptr(q_kvlen),
                                  ptr(q_kvstart), ptr(tree_mask), ptr(page_indptr), ptr(page_indices),
                                  c_int(t), c_int(q.stride(0)), c_int(hq), c_int(hkv), c_int(d),
                                  c_int(page), c_int(sink), c_float(sm_scale), c_float(softcap),
                                  c_int(DTYPE_CODE[q.dtype]), stream_ptr())
        check(rc, "mlcb_attn_simt")
    return (out, lse) if return_lse else out


def mla_append(rows: torch.Tensor, cache: torch.Tensor, slot: torch.Tensor, page: int) -> None:
    """Latent-attention cache write: row ``t`` of ``rows [T, D]`` (= [rotated rotary key | normalised latent]) goes
    to slot ``slot[t]`` of one layer's cache ``[num_pages, 1, 1, page, D]`` (reference: ``append_mla_kv``,
    ``python/mlc_llm/model/deepseek_v2/deepseek_v2_model.py:338-344``)."""
    if not rows.is_cuda:
        ref.mla_append(rows, cache, slot, page)
        return
    assert rows.is_contiguous() and cache.is_contiguous() and rows.dtype == cache.dtype
    rc = lib().mlcb_mla_append(ptr(rows), ptr(cache), ptr(slot), c_int(rows.shape[0]), c_int(rows.shape[1]),
                               c_ll(cache.shape[0] * page), c_int(DTYPE_CODE[rows.dtype]),
                               ptr(status_word(rows.device)), stream_ptr())
    check(rc, "mlcb_mla_append")


def mla_attention(q: torch.Tensor, cache: torch.Tensor, q_seq: torch.Tensor, q_kvlen: torch.Tensor,
                  page_indptr: torch.Tensor, page_indices: torch.Tensor, rope: int, rank: int, page: int,
                  sm_scale: float, q_kvstart: Optional[torch.Tensor] = None, sink: int = 0,
                  tree_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Latent attention in its absorbed form: ``q [T, hq, rope + rank]`` (per head: rotated rotary part, then the
    no-position part already multiplied by the key up-projection) against the compressed cache, whose one row per
    token is shared by all heads. Returns the attention-weighted latents ``[T, hq, rank]``; the caller applies the
    value up-projection (reference: the absorbed ``cross_attention`` of the MLA cache,
    ``python/mlc_llm/model/deepseek_v2/deepseek_v2_model.py:346-385``)."""
    t, hq, d = q.shape
    if not q.is_cuda:
        return ref.mla_attention(q, cache, q_seq, q_kvlen, page_indptr, page_indices, rope, rank, page, sm_scale,
                                 q_kvstart, sink, tree_mask)
    assert q.is_contiguous() and cache.is_contiguous() and q.dtype == cache.dtype and d == rope + rank
    out = torch.empty(t, hq, rank, dtype=q.dtype, device=q.device)
    rc = lib().mlcb_attn_mla(ptr(q), ptr(cache), ptr(out), ptr(q_seq), ptr(q_kvlen), ptr(q_kvstart), ptr(tree_mask),
                             ptr(page_indptr), ptr(page_indices), c_int(t), c_int(hq * d), c_int(hq), c_int(rope),
                             c_int(rank), c_int(page), c_int(cache.shape[0]), c_int(sink), c_float(sm_scale),
                             c_int(DTYPE_CODE[q.dtype]), ptr(status_word(q.device)), stream_ptr())
    if rc == -1:
        raise ValueError(f"latent attention kernel: rope {rope} and rank {rank} must be multiples of 64 with "
                         f"rope + rank <= 576, in fp16 or bf16")
    check(rc, "mlcb_attn_mla")
    return out


def encoder_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, key_lens: Optional[torch.Tensor] = None,
                      causal: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """Attention over whole sequences (vision towers, BERT-style encoders). ``q``, ``k``, ``v``: ``[B, S, H, D]``
    views (last dimension contiguous); ``key_lens``: int32 ``[B]`` number of valid keys per batch entry.
    Returns a contiguous ``[B, S, H, D]`` tensor."""
    b, s, h, d = q.shape
    scale = float(scale) if scale is not None else d ** -0.5
    if q.is_cuda and q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype and v.dtype == q.dtype \
            and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and k.shape == q.shape == v.shape:
        out = torch.empty(b, s, h, d, dtype=q.dtype, device=q.device)
        kl = None if key_lens is None else key_lens.to(torch.int32).contiguous()
        ll = ctypes.c_longlong
        rc = lib().mlcb_attn_encoder(ptr(q), ptr(k), ptr(v), ptr(out), ptr(kl), c_int(b), c_int(s), c_int(h), c_int(d),
                                     ll(q.stride(0)), ll(q.stride(1)), ll(q.stride(2)), ll(k.stride(0)),
                                     ll(k.stride(1)), ll(k.stride(2)), ll(v.stride(0)), ll(v.stride(1)),
                                     ll(v.stride(2)), c_float(scale), c_int(1 if causal else 0),
                                     c_int(DTYPE_CODE[q.dtype]), stream_ptr())
        if rc == 0:
            return out
        if rc > 0:
            check(rc, "mlcb_attn_encoder")
    # head dims the kernel does not have, fp32, CPU: tensor operations in fp32
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    att = (qf @ kf.transpose(-1, -2)) * scale
    if key_lens is not None:
        pad = torch.arange(s, device=q.device)[None, :] >= key_lens.to(q.device)[:, None]
        att = att.masked_fill(pad[:, None, None, :], float("-inf"))
    if causal:
        att = att.masked_fill(torch.ones(s, s, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    return (torch.softmax(att, dim=-1) @ vf).transpose(1, 2).to(q.dtype).contiguous()


# --------------------------------------------------------------------------- logits / sampling
def softmax_temperature(logits: torch.Tensor, temperature: torch.Tensor, active_vocab: int = 0):
    if not logits.is_cuda:
        return ref.softmax_temperature(logits, temperature, active_vocab)
    probs = torch.empty_like(logits)
    rc = lib().mlcb_softmax_temperature(ptr(logits), ptr(probs), ptr(temperature),
                                        c_int(logits.shape[0]), c_int(logits.shape[1]),
                                        c_int(active_vocab), stream_ptr())
    check(rc, "mlcb_softmax_temperature")
    return probs


def argmax(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return torch.argmax(x, dim=-1).to(torch.int32)
    out = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    rc = lib().mlcb_argmax(ptr(x), ptr(out), ptr(None), c_int(x.shape[0]), c_int(x.shape[1]),
                           stream_ptr())
    check(rc, "mlcb_argmax")
    return out


def apply_logit_bias(logits, pos2seq, token, bias) -> None:
    if not logits.is_cuda:
        return ref.apply_logit_bias(logits, pos2seq, token, bias)
    rc = lib().mlcb_logit_bias(ptr(logits), ptr(pos2seq), ptr(token), ptr(bias),
                               c_int(token.shape[0]), c_int(logits.shape[1]), stream_ptr())
    check(rc, "mlcb_logit_bias")


def apply_penalty(logits, pos2seq, token, cnt, penalties) -> None:
    if not logits.is_cuda:
        return ref.apply_penalty(logits, pos2seq, token, cnt, penalties)
    rc = lib().mlcb_penalty(ptr(logits), ptr(pos2seq), ptr(token), ptr(cnt), ptr(penalties),
                            c_int(token.shape[0]), c_int(logits.shape[1]), stream_ptr())
    check(rc, "mlcb_penalty")


def apply_bitmask(logits, rows, bitmask) -> None:
    if not logits.is_cuda:
        return ref.apply_bitmask(logits, rows, bitmask)
    rc = lib().mlcb_bitmask(ptr(logits), ptr(rows), ptr(bitmask), c_int(rows.shape[0]),
                            c_int(logits.shape[1]), stream_ptr())
    check(rc, "mlcb_bitmask")


def sample(probs, rows, uniform, top_p, top_k=None):
    """Returns (token ids int32 [n], renormalised prob of each sampled token fp32 [n])."""
    if not probs.is_cuda:
        return ref.sample(probs, rows, uniform, top_p, top_k)
    n = uniform.shape[0]
    tok = torch.empty(n, dtype=torch.int32, device=probs.device)
    pr = torch.empty(n, dtype=torch.float32, device=probs.device)
    rc = lib().mlcb_sample(ptr(probs), ptr(rows), ptr(uniform), ptr(top_p), ptr(top_k), ptr(tok),
                           ptr(pr), c_int(n), c_int(probs.shape[1]), stream_ptr())
    check(rc, "mlcb_sample")
    return tok, pr


def renorm_top_p(probs, rows, top_p) -> None:
    if not probs.is_cuda:
        return ref.renorm_top_p(probs, rows, top_p)
    rc = lib().mlcb_renorm_top_p(ptr(probs), ptr(rows), ptr(top_p), c_int(top_p.shape[0]),
                                 c_int(probs.shape[1]), stream_ptr())
    check(rc, "mlcb_renorm_top_p")


def take_probs(probs, rows, token, k: int):
    if not probs.is_cuda:
        return ref.take_probs(probs, rows, token, k)
    n = token.shape[0]
    outp = torch.empty(n, dtype=torch.float32, device=probs.device)
    tp = torch.empty(n, max(k, 1), dtype=torch.float32, device=probs.device)
    ti = torch.empty(n, max(k, 1), dtype=torch.int32, device=probs.device)
    rc = lib().mlcb_take_probs(ptr(probs), ptr(rows), ptr(token), ptr(outp), ptr(tp), ptr(ti),
                               c_int(n), c_int(k), c_int(probs.shape[1]), stream_ptr())
    check(rc, "mlcb_take_probs")
    return outp, tp[:, :k], ti[:, :k]


def verify_tree(draft_probs, draft_tokens, model_probs, first_child, next_sibling, uniform,
                parent_ptr) -> None:
    if not model_probs.is_cuda:
        return ref.verify_tree(draft_probs, draft_tokens, model_probs, first_child, next_sibling,
                               uniform, parent_ptr)
    rc = lib().mlcb_verify_tree(ptr(draft_probs), ptr(draft_tokens), ptr(model_probs),
                                ptr(first_child), ptr(next_sibling), ptr(uniform), ptr(parent_ptr),
                                c_int(parent_ptr.shape[0]), c_int(model_probs.shape[1]),
                                c_int(draft_tokens.shape[0] + 1), stream_ptr())
    check(rc, "mlcb_verify_tree")


def row_gather(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    if not src.is_cuda:
        return src[idx.long()].clone()
    out = torch.empty(idx.shape[0], *src.shape[1:], dtype=src.dtype, device=src.device)
    row_bytes = src[0].numel() * src.element_size()
    rc = lib().mlcb_row_copy(ptr(src), ptr(out), ptr(idx), c_int(idx.shape[0]), c_int(row_bytes),
                             c_int(0), stream_ptr())
    check(rc, "mlcb_row_copy")
    return out


def row_scatter(dst: torch.Tensor, idx: torch.Tensor, src: torch.Tensor) -> None:
    if not dst.is_cuda:
        dst[idx.long()] = src
        return
    row_bytes = dst[0].numel() * dst.element_size()
    rc = lib().mlcb_row_copy(ptr(src), ptr(dst), ptr(idx), c_int(idx.shape[0]), c_int(row_bytes),
                             c_int(1), stream_ptr())
    check(rc, "mlcb_row_copy")


# --------------------------------------------------------------------------- mixture of experts
def moe_router(logits: torch.Tensor, k: int, renorm: bool = True):
    """Softmax over the experts, top-k, optional renormalisation. Returns (weights fp32 [T, k],
    expert ids int32 [T, k])."""
    if not logits.is_cuda:
        return ref.moe_softmax_topk(logits, k, renorm)
    t, e = logits.shape
    w = torch.empty(t, k, dtype=torch.float32, device=logits.device)
    idx = torch.empty(t, k, dtype=torch.int32, device=logits.device)
    lg = logits.contiguous()
    rc = lib().mlcb_moe_router(ptr(lg), ptr(w), ptr(idx), c_int(t), c_int(e), c_int(k), c_int(0),
                               c_int(1 if renorm else 0), c_int(DTYPE_CODE[lg.dtype]), stream_ptr())
    check(rc, "mlcb_moe_router")
    return w, idx


def moe_permute(experts: torch.Tensor, num_experts: int):
    """Expert-major ordering of the (token, slot) pairs. Returns (offsets int32 [E+1], sorted_pos
    int32 [T*k] = row of each pair, src_token int32 [T*k] = token feeding each row)."""
    t, k = experts.shape
    n = t * k
    if not experts.is_cuda:
        flat = experts.reshape(-1).long()
        order = torch.sort(flat, stable=True).indices
        sorted_pos = torch.empty(n, dtype=torch.int32)
        sorted_pos[order] = torch.arange(n, dtype=torch.int32)
        counts = torch.bincount(flat, minlength=num_experts)
        offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
        offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
        return offsets, sorted_pos, (order // k).to(torch.int32)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=experts.device)
    sorted_pos = torch.empty(n, dtype=torch.int32, device=experts.device)
    src_token = torch.empty(n, dtype=torch.int32, device=experts.device)
    rc = lib().mlcb_moe_permute(ptr(experts.contiguous()), c_int(n), c_int(k), c_int(num_experts), ptr(offsets),
                                ptr(sorted_pos), ptr(src_token), stream_ptr())
    check(rc, "mlcb_moe_permute")
    return offsets, sorted_pos, src_token


def grouped_linear(x: torch.Tensor, lw: LinearWeight, offsets: torch.Tensor,
                   out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Rows ``[offsets[e], offsets[e+1])`` of ``x`` times expert ``e``'s weight ``lw.w[e]``."""
    od = out_dtype or x.dtype
    e = lw.w.shape[0]
    n = lw.w.shape[1]
    if not x.is_cuda:
        y = torch.zeros(x.shape[0], n, dtype=od)
        w = lw.dense(torch.float32)
        off = offsets.tolist()
        for i in range(e):
            if off[i + 1] > off[i]:
                y[off[i]:off[i + 1]] = ref.linear_dense(x[off[i]:off[i + 1]], w[i], None, od)
        return y
    rows, k = x.shape
    y = torch.empty(rows, n, dtype=od, device=x.device)
    if rows == 0:
        return y
    x2 = x if x.stride(-1) == 1 else x.contiguous()
    if lw.kind in ("fp8_block", "fp8_tensor") and lw.w.dtype == torch.float8_e4m3fn and k % 128 == 0 \
            and n % 128 == 0 and x.dtype in (torch.float16, torch.bfloat16):
        # expert weights stay fp8 in memory; the kernel expands them tile by tile
        scale = _expert_block_scale(lw)
        rc = lib().mlcb_gemm_grouped_fp8(ptr(x2), ptr(lw.w), ptr(scale), ptr(y), ptr(offsets), ptr(None), ptr(None),
                                         c_int(e), c_int(e), c_int(rows), c_int(rows), c_int(n), c_int(k),
                                         c_int(x2.stride(0)), c_int(n), c_int(DTYPE_CODE[x.dtype]),
                                         c_int(DTYPE_CODE[od]), ptr(status_word(x.device)), stream_ptr())
        check(rc, f"mlcb_gemm_grouped_fp8(rows={rows},E={e},N={n},K={k})")
        return y
    if rows <= _MOE_GEMV_MAX_ROWS and lw.kind == "q4" and lw.device_layout and x.dtype == torch.float16 \
            and lw.scale is not None and lw.scale.dtype == torch.float16 and k % 32 == 0 \
            and lw.quant is not None and lw.quant.bits == 4 and lw.quant.group_size == 32 \
            and od in (torch.float16, torch.float32):
        # a handful of (token, expert) pairs (single-stream decode): memory-bound GEMV over the experts in use;
        # the expert of every row follows from the offsets without leaving the device
        slab = torch.searchsorted(offsets[1:].contiguous(), torch.arange(rows, device=x.device, dtype=offsets.dtype),
                                  right=True).to(torch.int32)
        rc = lib().mlcb_gemv_q4_grouped(ptr(x2), ptr(lw.w), ptr(lw.scale), ptr(y), ptr(slab), c_int(rows), c_int(n),
                                        c_int(k), c_int(x2.stride(0)), c_int(n), c_int(DTYPE_CODE[od]), stream_ptr())
        if rc == 0:
            return y
        if rc > 0:
            check(rc, "mlcb_gemv_q4_grouped")
    q4 = lw.q4_tileable(k) and x.dtype == lw.scale.dtype
    w = lw.q4_tiles() if q4 else (lw.w if lw.kind == "dense" else lw.dense(x.dtype))
    rc = lib().mlcb_gemm_grouped(ptr(x2), ptr(w), ptr(w) if q4 else ptr(None), ptr(y), ptr(offsets),
                                 c_int(e), c_int(rows), c_int(n), c_int(k), c_int(x2.stride(0)), c_int(n),
                                 c_int(DTYPE_CODE[x.dtype]), c_int(DTYPE_CODE[od]), ptr(status_word(x.device)),
                                 stream_ptr())
    check(rc, f"mlcb_gemm_grouped(rows={rows},E={e},N={n},K={k})")
    return y


def _expert_block_scale(lw: LinearWeight) -> torch.Tensor:
    """fp32 block scales ``[E, N / 128, K / 128]`` of stacked fp8 expert weights (a per-tensor scale per expert, or
    one for all, is repeated over the grid)."""
    if lw.kind == "fp8_block":
        if lw.scale.dtype != torch.float32 or not lw.scale.is_contiguous():
            lw.scale = lw.scale.float().contiguous()
        return lw.scale
    if lw._block_scale is None:
        e, n, k = lw.w.shape
        per_expert = lw.scale.float().reshape(-1)
        per_expert = per_expert if per_expert.numel() == e else per_expert[:1].expand(e)
        lw._block_scale = per_expert.view(e, 1, 1).expand(e, n // 128, k // 128).contiguous()
    return lw._block_scale


def moe_combine(y: torch.Tensor, weights: torch.Tensor, sorted_pos: torch.Tensor,
                add: Optional[torch.Tensor]) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * y[sorted_pos[t * k + j]] (+ add[t])``."""
    t, k = weights.shape
    if not y.is_cuda:
        rows = y[sorted_pos.long()].float().view(t, k, -1)
        out = (rows * weights.float().unsqueeze(-1)).sum(1)
        if add is not None:
            out = out + add.float()
        return out.to(y.dtype)
    out = torch.empty(t, y.shape[1], dtype=y.dtype, device=y.device)
    if weights.dtype != torch.float32 or not weights.is_contiguous():
        weights = weights.float().contiguous()  # the kernel reads fp32 routing weights
    rc = lib().mlcb_moe_combine(ptr(y), ptr(weights), ptr(sorted_pos), ptr(add), ptr(out), c_int(t),
                                c_int(y.shape[1]), c_int(k), c_int(DTYPE_CODE[y.dtype]), stream_ptr())
    check(rc, "mlcb_moe_combine")
    return out


__all__ = [n for n in dir() if not n.startswith("_")]
