"""Fused tensor-parallel collectives: the host side of ``mlcb_gemm_fused``.

One object per tensor-parallel group owns the symmetric peer buffers and the call counter (epoch)
that the kernels' flags carry.  The counter is kept in device memory as a per-forward base plus the
call's index inside the forward (a launch argument): a forward that was captured into a CUDA graph
replays with fresh call numbers because only the base changes (``mlcb_epoch_add`` at the end of the
forward is part of the graph).  Ranks stay in step because all of them run the same forwards.

* ``gemm_rs_norm``  row-parallel GEMM (``o_proj`` / ``down_proj``) whose epilogue pushes partial sums
  to the rows' owners and whose tail does reduce + residual add + RMSNorm + all-gather of the
  normalised rows — one launch instead of GEMM, all-reduce, add and RMSNorm.
* ``gemm_ag``       column-parallel GEMM (``qkv_proj`` / ``gate_up_proj``) reading the gathered rows,
  starting on the rows that have arrived.

The residual stream stays scattered: each rank keeps only the rows it owns.  The NCCL all-reduce
path (``Communicator.all_reduce``) stays available as the baseline and as the numerics oracle.

Reference behaviour being replaced: ``op.ccl_allreduce(out, "sum") + residual`` after attention and
after the MLP (``model/llama/llama_model.py:211-214``) followed by the fused add+RMSNorm
(``compiler_pass/fuse_add_norm.py``).
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..ops import LinearWeight, _gemm_scratch
from ..ops._lib import DTYPE_CODE, check, lib, ptr, status_word, stream_ptr
from .symm import LocalBuffer, SymmetricBuffer


class FusedArgs(ctypes.Structure):
    """Mirror of ``MlcbFusedArgs`` in ``csrc/kernels/gemm_tcgen05.cu``."""

    _fields_ = [
        ("rs_world", ctypes.c_int), ("rs_rank", ctypes.c_int), ("rs_rows", ctypes.c_int),
        ("rs_epoch", ctypes.c_int),
        ("rs_recv", ctypes.c_void_p), ("rs_flag", ctypes.c_void_p),
        ("rs_count", ctypes.c_void_p), ("rs_residual", ctypes.c_void_p), ("rs_norm_w", ctypes.c_void_p),
        ("rs_eps", ctypes.c_float), ("rs_w_offset", ctypes.c_float),
        ("ag_xn", ctypes.c_void_p), ("ag_flag", ctypes.c_void_p),
        ("ag_wait", ctypes.c_void_p), ("ag_epoch", ctypes.c_int), ("reserved", ctypes.c_int),
        ("epoch_base", ctypes.c_void_p),
        ("ar_world", ctypes.c_int), ("ar_rank", ctypes.c_int), ("ar_epoch", ctypes.c_int), ("ar_pad", ctypes.c_int),
        ("ar_mc", ctypes.c_void_p), ("ar_peers", ctypes.c_void_p), ("ar_flags", ctypes.c_void_p),
        ("ar_counter", ctypes.c_void_p), ("ar_xn", ctypes.c_void_p),
    ]


def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


class FusedCollectives:
    """Symmetric buffers + launch helpers for one tensor-parallel group."""

    def __init__(self, hidden: int, dtype: torch.dtype, max_tokens: int, device: torch.device,
                 group=None, world_size: int = 1, mode: Optional[str] = None):
        assert dtype in (torch.float16, torch.bfloat16)
        self.hidden, self.dtype, self.device = hidden, dtype, device
        # "ar": GEMM + in-kernel all-reduce through NVSwitch multicast loads (+ residual + RMSNorm), every
        # rank keeps the whole residual stream; "rs": the reduce-scatter / all-gather pair of kernels with
        # peer stores, residual rows scattered over the ranks
        self.mode = mode or os.environ.get("MLCB_FUSED_TP_MODE", "ar")
        if self.mode not in ("ar", "rs"):
            raise ValueError(f"unknown fused tensor-parallel mode {self.mode!r}")
        if self.mode == "ar":
            self._init_ar(max_tokens, group, world_size)
            return
        esize = 2
        self.rows_cap = _round_up(-(-max_tokens // max(1, world_size)), 32)
        world = max(1, world_size)
        recv_bytes = world * self.rows_cap * hidden * esize          # one parity
        flag_bytes = _round_up((self.rows_cap // 32) * world * 4, 256)
        xn_bytes = world * self.rows_cap * hidden * esize
        ag_flag_bytes = _round_up(world * self.rows_cap // 8 * 4, 256)
        self.off_recv = [0, recv_bytes]
        self.off_flag = 2 * recv_bytes
        self.off_xn = self.off_flag + flag_bytes
        self.off_agflag = self.off_xn + xn_bytes
        total = self.off_agflag + ag_flag_bytes
        if world > 1:
            self.buf = SymmetricBuffer(total, group, device)
        else:
            self.buf = LocalBuffer(total, device)
        self.world, self.rank = self.buf.world_size, self.buf.rank
        assert self.world == world
        # peer address tables: [recv parity 0][recv parity 1][rs flags][xn][ag flags], 8 slots each
        table = torch.zeros(5, 8, dtype=torch.int64)
        for r in range(self.world):
            table[0, r] = self.buf.peer_ptr(r, self.off_recv[0])
            table[1, r] = self.buf.peer_ptr(r, self.off_recv[1])
            table[2, r] = self.buf.peer_ptr(r, self.off_flag)
            table[3, r] = self.buf.peer_ptr(r, self.off_xn)
            table[4, r] = self.buf.peer_ptr(r, self.off_agflag)
        self.table = table.to(device)
        self.rs_count = torch.zeros(world * self.rows_cap // 32 + 8, dtype=torch.int32, device=device)
        self.residual = torch.zeros(self.rows_cap, hidden, dtype=dtype, device=device)
        self.epoch_dev = torch.zeros(4, dtype=torch.int32, device=device)  # [0]: base of the call numbers
        self.base = 0        # host mirror of epoch_dev[0] once every queued forward has run
        self.call = 0        # reduce-scatter calls since begin()
        self.rows = self.rows_cap
        self.tokens = 0
        self.launches = 0

    # ------------------------------------------------------------------ all-reduce form
    def _init_ar(self, max_tokens: int, group, world_size: int) -> None:
        hidden, esize = self.hidden, 2
        world = max(1, world_size)
        self.rows_cap = _round_up(-(-max_tokens // world), 32)
        cap = world * self.rows_cap
        part_bytes = _round_up(cap * hidden * esize, 4096)           # one parity
        self.off_part = [0, part_bytes]
        self.off_arflag = 2 * part_bytes
        total = self.off_arflag + 256
        self.buf = SymmetricBuffer(total, group, self.device) if world > 1 else LocalBuffer(total, self.device)
        self.world, self.rank = self.buf.world_size, self.buf.rank
        assert self.world == world
        # peer address tables: [partial sums parity 0][parity 1][arrival flags], 8 slots each
        table = torch.zeros(3, 8, dtype=torch.int64)
        for r in range(self.world):
            table[0, r] = self.buf.peer_ptr(r, self.off_part[0])
            table[1, r] = self.buf.peer_ptr(r, self.off_part[1])
            table[2, r] = self.buf.peer_ptr(r, self.off_arflag)
        self.table = table.to(self.device)
        self.ar_counter = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.residual = torch.zeros(cap, hidden, dtype=self.dtype, device=self.device)
        self.xn_local = torch.zeros(cap, hidden, dtype=self.dtype, device=self.device)
        self.epoch_dev = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.base = self.call = 0
        self.rows = self.rows_cap
        self.tokens = 0
        self.launches = 0
        self.multimem = self.buf.mc_ptr != 0

    def gemm_ar_norm(self, x: torch.Tensor, lw: LinearWeight, norm_w: torch.Tensor, eps: float,
                     w_offset: float = 0.0) -> torch.Tensor:
        """``residual += sum_ranks(x @ W^T)`` on every rank; returns ``rmsnorm(residual)`` ``[tokens, hidden]``
        in local memory. One launch: the GEMM stores this rank's partial sums in its copy of a symmetric
        buffer, the kernel's tail waits for all ranks and reduces through the multicast mapping."""
        assert self.mode == "ar" and x.shape[0] == self.tokens and x.is_contiguous()
        n = lw.out_features or lw.w.shape[0]
        assert n == self.hidden
        self.call += 1
        parity = self.epoch & 1
        a = FusedArgs()
        a.ar_world, a.ar_rank, a.ar_epoch = self.world, self.rank, self.call
        a.epoch_base = self.epoch_dev.data_ptr()
        a.ar_mc = (self.buf.mc_ptr + self.off_part[parity]) if self.multimem else None
        a.ar_peers = self.table[parity].data_ptr()
        a.ar_flags = self.table[2].data_ptr()
        a.ar_counter = self.ar_counter.data_ptr()
        a.ar_xn = self.xn_local.data_ptr()
        a.rs_residual = self.residual.data_ptr()
        a.rs_norm_w = norm_w.data_ptr()
        a.rs_eps, a.rs_w_offset = float(eps), float(w_offset)
        y = self.buf.view(self.off_part[parity], (self.world * self.rows_cap, self.hidden), self.dtype)[: self.tokens]
        # a bias of a row-parallel layer is added once, by rank 0
        self._launch(x, lw, y, n, x.dtype, a, bias=self.rank == 0 and lw.bias is not None)
        return self.xn_local[: self.tokens]

    # ------------------------------------------------------------------ per-forward state
    def begin(self, tokens: int) -> None:
        """Fix the row partition of this forward call (every rank passes the same token count)."""
        self.end()
        if tokens > self.rows_cap * self.world:
            raise ValueError(f"{tokens} tokens exceed the fused-collective buffers "
                             f"({self.rows_cap * self.world}); raise prefill_chunk_size-based capacity")
        self.tokens = tokens
        self.rows = _round_up(-(-tokens // self.world), 32)

    def end(self) -> None:
        """Close a forward: the device-side base moves past the call numbers it used."""
        if self.call:
            rc = lib().mlcb_epoch_add(ptr(self.epoch_dev), ctypes.c_int(self.call), stream_ptr())
            check(rc, "mlcb_epoch_add")
            self.base += self.call
            self.call = 0
            self.launches += 1

    def note_replay(self, calls: int) -> None:
        """A captured forward with ``calls`` reduce-scatter launches was replayed."""
        self.base += calls

    @property
    def epoch(self) -> int:
        """Number of the latest reduce-scatter call."""
        return self.base + self.call

    def owned(self) -> range:
        lo = min(self.tokens, self.rank * self.rows)
        return range(lo, min(self.tokens, lo + self.rows))

    def scatter_residual(self, x: torch.Tensor) -> None:
        """Start of a forward: this rank's rows of the (replicated) embedding output become its part
        of the residual stream."""
        if self.mode == "ar":
            self.residual[: self.tokens].copy_(x)
            return
        own = self.owned()
        if len(own):
            self.residual[: len(own)].copy_(x[own.start: own.stop])

    def xn(self) -> torch.Tensor:
        """This rank's gather buffer, ``[tokens, hidden]``."""
        return self.buf.view(self.off_xn, (self.world * self.rows_cap, self.hidden), self.dtype)[: self.tokens]

    def _ag_flags_ptr(self) -> int:
        return self.buf.peer_ptr(self.rank, self.off_agflag)

    # ------------------------------------------------------------------ launches
    def _launch(self, x: torch.Tensor, lw: LinearWeight, y: Optional[torch.Tensor], n: int, od: torch.dtype,
                args: FusedArgs, bias: bool) -> None:
        m, k = x.shape
        q4 = lw.q4_tileable(k) and x.dtype == lw.scale.dtype
        w = lw.q4_tiles() if q4 else lw.dense(x.dtype)
        rc = lib().mlcb_gemm_fused(
            ptr(x), ptr(w), ptr(w) if q4 else ptr(None), ptr(lw.bias) if bias else ptr(None), ptr(y),
            ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), ctypes.c_int(x.stride(0)), ctypes.c_int(n),
            ctypes.c_int(DTYPE_CODE[x.dtype]), ctypes.c_int(DTYPE_CODE[od]), ptr(status_word(x.device)),
            *_gemm_scratch(x.device), ctypes.byref(args), stream_ptr())
        check(rc, f"mlcb_gemm_fused(M={m},N={n},K={k})")
        self.launches += 1

    def gemm_rs_norm(self, x: torch.Tensor, lw: LinearWeight, norm_w: torch.Tensor, eps: float,
                     w_offset: float = 0.0) -> torch.Tensor:
        """``residual[own rows] += sum_ranks(x @ W^T)``; returns the gather buffer that will hold
        ``rmsnorm(residual)`` for all rows once the peers' pushes have landed (consume it with
        :meth:`gemm_ag` or after :meth:`wait_gather`)."""
        assert x.shape[0] == self.tokens and x.is_contiguous()
        n = lw.out_features or lw.w.shape[0]
        assert n == self.hidden
        self.call += 1
        a = FusedArgs()
        a.rs_world, a.rs_rank, a.rs_rows, a.rs_epoch = self.world, self.rank, self.rows, self.call
        a.epoch_base = self.epoch_dev.data_ptr()
        # the receive buffer alternates with the call number; a captured forward keeps the parity it
        # was captured with, which holds as long as every forward makes an even number of these calls
        a.rs_recv = self.table[self.epoch & 1].data_ptr()
        a.rs_flag = self.table[2].data_ptr()
        a.rs_count = self.rs_count.data_ptr()
        a.rs_residual = self.residual.data_ptr()
        a.rs_norm_w = norm_w.data_ptr()
        a.rs_eps, a.rs_w_offset = float(eps), float(w_offset)
        a.ag_xn = self.table[3].data_ptr()
        a.ag_flag = self.table[4].data_ptr()
        a.ag_wait, a.ag_epoch = None, 0
        # a bias of a row-parallel layer is added once, by rank 0
        self._launch(x, lw, None, n, x.dtype, a, bias=self.rank == 0 and lw.bias is not None)
        return self.xn()

    def gemm_ag(self, lw: LinearWeight, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``gathered rows @ W^T`` where the rows are the output of the latest :meth:`gemm_rs_norm`."""
        x = self.xn()
        n = lw.out_features or lw.w.shape[0]
        od = out_dtype or x.dtype
        y = torch.empty(self.tokens, n, dtype=od, device=self.device)
        a = FusedArgs()
        a.ag_wait, a.ag_epoch = self._ag_flags_ptr(), self.call
        a.epoch_base = self.epoch_dev.data_ptr()
        self._launch(x, lw, y, n, od, a, bias=lw.bias is not None)
        return y

    def wait_gather(self) -> torch.Tensor:
        """Make the gather buffer safe to read for any later kernel on this stream."""
        rc = lib().mlcb_flag_wait(ctypes.c_void_p(self._ag_flags_ptr()), ctypes.c_int(self.tokens),
                                  ctypes.c_int(self.call), ptr(self.epoch_dev), ptr(status_word(self.device)),
                                  stream_ptr())
        check(rc, "mlcb_flag_wait")
        return self.xn()
