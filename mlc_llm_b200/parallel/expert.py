"""Expert parallelism for mixture-of-experts layers: all-to-all token dispatch and result combine over
symmetric peer buffers (kernels in ``csrc/kernels/moe_ep.cu``), expert matmuls on the table-driven
grouped tcgen05 GEMM.

Every rank owns ``E / world`` whole experts and a contiguous slice of the batch's tokens.  One layer:

1. ``moe_permute`` orders this rank's (token, slot) pairs by expert (hence by destination rank);
2. ``mlcb_ep_dispatch`` writes each pair's hidden row into the destination's receive region, plus the
   per-expert counts and the pair ids, then raises this rank's flag at every destination;
3. ``mlcb_ep_build_groups`` (receiver) waits for all senders and builds the table of received segments,
   ``mlcb_ep_compact`` copies them expert-major into one contiguous buffer (one GEMM group per local expert:
   an expert's weights are streamed once per exchange, not once per sender);
4. two grouped GEMMs with the activation in between run on the received rows;
5. ``mlcb_ep_combine_send`` sends each output row to its pair's slot on *every* rank;
6. every rank waits for all expert ranks and takes the weighted sum over the k slots of all tokens (the
   attention that follows is tensor parallel and wants every token on every rank, so no gather follows).

Call numbers (the epochs the flags carry) live in device memory and the last kernel of an exchange moves
them on, so a forward with these exchanges inside can be captured in a CUDA graph and replayed; nothing in the
exchange is an NCCL call.

The reference shards experts over their width instead (``model/mixtral/mixtral_model.py:144-145``)
and has no all-to-all; that layout remains available (``expert_parallel=False``) and is the numerics
oracle for this path.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops._lib import DTYPE_CODE, check, lib, ptr, status_word, stream_ptr
from .symm import LocalBuffer, SymmetricBuffer


class EpArgs(ctypes.Structure):
    """Mirror of ``MlcbEpArgs``."""

    _fields_ = [
        ("world", ctypes.c_int), ("rank", ctypes.c_int), ("e_local", ctypes.c_int), ("k", ctypes.c_int),
        ("hidden", ctypes.c_int), ("cap", ctypes.c_int), ("epoch", ctypes.c_int), ("pairs", ctypes.c_int),
        ("disp_x", ctypes.c_void_p), ("disp_meta", ctypes.c_void_p), ("disp_pair", ctypes.c_void_p),
        ("disp_flag", ctypes.c_void_p), ("comb_y", ctypes.c_void_p), ("comb_flag", ctypes.c_void_p),
        ("done_counter", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("epoch_base", ctypes.c_void_p), ("pair_base", ctypes.c_int),
    ]


def _up(v: int, m: int = 256) -> int:
    return (v + m - 1) // m * m


class ExpertParallel:
    """Buffers and launch sequence of the expert-parallel FFN for one process group."""

    def __init__(self, num_experts: int, top_k: int, hidden: int, dtype: torch.dtype, max_tokens: int,
                 device: torch.device, group=None, world_size: int = 1):
        assert dtype in (torch.float16, torch.bfloat16)
        world = max(1, world_size)
        if num_experts % world:
            raise ValueError(f"{num_experts} experts cannot be split over {world} ranks")
        self.E, self.k, self.hidden, self.dtype, self.device = num_experts, top_k, hidden, dtype, device
        self.e_local = num_experts // world
        self.tokens_cap = -(-max_tokens // world)          # tokens of one rank's slice
        self.cap = _up(self.tokens_cap * top_k, 32)        # rows one sender may route to one receiver
        es = 2
        x_bytes = _up(world * self.cap * hidden * es)
        meta_bytes = _up(world * (self.e_local + 1) * 4)
        pair_bytes = _up(world * self.cap * 4)
        comb_bytes = _up(world * self.tokens_cap * top_k * hidden * es)   # the pairs of all ranks
        # two parities of every data region, one set of flags
        self.off = {}
        cur = 0
        for name, size in (("x0", x_bytes), ("x1", x_bytes), ("meta0", meta_bytes), ("meta1", meta_bytes),
                           ("pair0", pair_bytes), ("pair1", pair_bytes), ("comb0", comb_bytes),
                           ("comb1", comb_bytes), ("dflag", 256), ("cflag", 256)):
            self.off[name] = cur
            cur += size
        self.buf = SymmetricBuffer(cur, group, device) if world > 1 else LocalBuffer(cur, device)
        self.world, self.rank, self.group = self.buf.world_size, self.buf.rank, group
        names = ["x0", "x1", "meta0", "meta1", "pair0", "pair1", "comb0", "comb1", "dflag", "cflag"]
        table = torch.zeros(len(names), 8, dtype=torch.int64)
        for i, n in enumerate(names):
            for r in range(self.world):
                table[i, r] = self.buf.peer_ptr(r, self.off[n])
        self.table = table.to(device)
        self.row = {n: i for i, n in enumerate(names)}
        self.done = torch.zeros(4, dtype=torch.int32, device=device)
        # one GEMM group per local expert over the compact (expert-major) copy of the received rows; the
        # received rows of an expert come as one segment per sender
        g = self.world * self.e_local
        self.group_begin = torch.zeros(self.e_local, dtype=torch.int32, device=device)
        self.group_count = torch.zeros(self.e_local, dtype=torch.int32, device=device)
        self.group_slab = torch.zeros(self.e_local, dtype=torch.int32, device=device)
        self.seg_src = torch.zeros(g, dtype=torch.int32, device=device)
        self.seg_dst = torch.zeros(g, dtype=torch.int32, device=device)
        self.seg_cnt = torch.zeros(g, dtype=torch.int32, device=device)
        self.live = torch.zeros(4, dtype=torch.int32, device=device)
        self.xc = torch.zeros(world * self.cap, hidden, dtype=dtype, device=device)
        self.pair_c = torch.zeros(world * self.cap, dtype=torch.int32, device=device)
        # number of finished exchanges: `epoch_dev` on the device (moved on by the last kernel of each
        # exchange), `base` its host mirror (which buffer parity the next exchange uses)
        self.epoch_dev = torch.zeros(4, dtype=torch.int32, device=device)
        self.base = 0
        self.launches = 0

    def token_slice(self, tokens: int) -> range:
        per = -(-tokens // self.world)
        lo = min(tokens, self.rank * per)
        return range(lo, min(tokens, lo + per))

    def note_replay(self, calls: int) -> None:
        """A captured forward with ``calls`` exchanges was replayed (the device counter moved by itself)."""
        self.base += calls

    def _args(self, pairs: int, pair_base: int) -> EpArgs:
        par = (self.base + 1) & 1
        a = EpArgs()
        a.world, a.rank, a.e_local, a.k = self.world, self.rank, self.e_local, self.k
        a.hidden, a.cap, a.epoch, a.pairs = self.hidden, self.cap, 1, pairs   # epoch: relative to *epoch_base
        a.epoch_base = self.epoch_dev.data_ptr()
        a.pair_base = pair_base
        a.disp_x = self.table[self.row[f"x{par}"]].data_ptr()
        a.disp_meta = self.table[self.row[f"meta{par}"]].data_ptr()
        a.disp_pair = self.table[self.row[f"pair{par}"]].data_ptr()
        a.disp_flag = self.table[self.row["dflag"]].data_ptr()
        a.comb_y = self.table[self.row[f"comb{par}"]].data_ptr()
        a.comb_flag = self.table[self.row["cflag"]].data_ptr()
        a.done_counter = self.done.data_ptr()
        a.status = status_word(self.device).data_ptr()
        return a

    def ffn(self, h: torch.Tensor, weights: torch.Tensor, experts: torch.Tensor, w13, w2,
            act: str = "silu") -> torch.Tensor:
        """Expert FFN of all tokens ``h [T, hidden]`` (replicated on the ranks) with routing ``weights /
        experts [T, k]``; this rank dispatches its slice of the tokens, runs its ``e_local`` experts (``w13 /
        w2``) on what it receives, and sums the outputs of all tokens. Returns ``[T, hidden]``."""
        total = h.shape[0]
        sl = self.token_slice(total)
        x, experts_own = h[sl.start: sl.stop], experts[sl.start: sl.stop]
        t = x.shape[0]
        if t > self.tokens_cap:
            raise ValueError(f"{t} tokens exceed the expert-parallel buffers ({self.tokens_cap} per rank)")
        par = (self.base + 1) & 1
        pairs = t * self.k
        a = self._args(pairs, sl.start * self.k)
        experts = experts_own
        dt = DTYPE_CODE[x.dtype]
        x = x.contiguous()
        if pairs:
            offsets, sorted_pos, _ = ops.moe_permute(experts.contiguous(), self.E)
        else:
            offsets = torch.zeros(self.E + 1, dtype=torch.int32, device=self.device)
            sorted_pos = torch.zeros(1, dtype=torch.int32, device=self.device)
            experts = torch.zeros(1, self.k, dtype=torch.int32, device=self.device)
        rc = lib().mlcb_ep_dispatch(ptr(x), ptr(experts), ptr(sorted_pos), ptr(offsets), ctypes.byref(a),
                                    ctypes.c_int(dt), stream_ptr())
        check(rc, "mlcb_ep_dispatch")
        a.done_counter = self.done[1:].data_ptr()
        rc = lib().mlcb_ep_build_groups(ctypes.byref(a), ptr(self.group_begin), ptr(self.group_count),
                                        ptr(self.group_slab), ptr(self.seg_src), ptr(self.seg_dst),
                                        ptr(self.seg_cnt), ptr(self.live), stream_ptr())
        check(rc, "mlcb_ep_build_groups")
        rows = self.world * self.cap
        recv = self.buf.view(self.off[f"x{par}"], (rows, self.hidden), self.dtype)
        pair_in = self.buf.peer_ptr(self.rank, self.off[f"pair{par}"])
        # expert-major compaction: each local expert's rows from all senders become one contiguous group, so its
        # weights are read once per exchange
        rc = lib().mlcb_ep_compact(ptr(recv), ptr(self.xc), ctypes.c_void_p(pair_in), ptr(self.pair_c),
                                   ptr(self.seg_src), ptr(self.seg_dst), ptr(self.seg_cnt), ptr(self.live),
                                   ctypes.c_int(self.world * self.e_local), ctypes.c_int(rows),
                                   ctypes.c_int(self.hidden), ctypes.c_int(dt), stream_ptr())
        check(rc, "mlcb_ep_compact")
        # buffers are sized for the worst case; the work is bounded by what can arrive in this exchange
        bound = min(rows, _up(total * self.k, 32))
        hint = max(1, min(bound, -(-total * self.k // self.world)))
        h1 = self._grouped(self.xc, w13, bound, hint)
        y = self._grouped(ops.act_mul(h1, act, live_rows=self.live), w2, bound, hint)
        a.done_counter = self.done[2:].data_ptr()
        rc = lib().mlcb_ep_combine_send(ptr(y), ptr(self.live), ptr(self.pair_c), ctypes.byref(a), ctypes.c_int(dt),
                                        stream_ptr())
        check(rc, "mlcb_ep_combine_send")
        flags = self.buf.peer_ptr(self.rank, self.off["cflag"])
        rc = lib().mlcb_ep_wait_flags(ctypes.c_void_p(flags), ctypes.c_int(self.world), ctypes.c_int(1),
                                      ptr(self.epoch_dev), ptr(status_word(self.device)), stream_ptr())
        check(rc, "mlcb_ep_wait_flags")
        self.base += 1
        self.launches += 7
        all_pairs = total * self.k
        comb = self.buf.view(self.off[f"comb{par}"], (self.world * self.tokens_cap * self.k, self.hidden),
                             self.dtype)[:all_pairs]
        ident = self._ident(all_pairs)
        return ops.moe_combine(comb, weights.contiguous(), ident, None)

    def _ident(self, n: int) -> torch.Tensor:
        """0 .. n-1 (the combine reads pair p of the buffer for pair p); one allocation, grown on demand."""
        cur = getattr(self, "_ident_buf", None)
        if cur is None or cur.numel() < n:
            cur = self._ident_buf = torch.arange(max(n, 4096), dtype=torch.int32, device=self.device)
        return cur[:n]

    def _grouped(self, x: torch.Tensor, lw, rows: int, hint: int) -> torch.Tensor:
        n, k = lw.w.shape[1], x.shape[1]
        if lw.kind in ("fp8_block", "fp8_tensor") and lw.w.dtype == torch.float8_e4m3fn and k % 128 == 0 \
                and n % 128 == 0:
            y = torch.empty(rows, n, dtype=x.dtype, device=x.device)
            rc = lib().mlcb_gemm_grouped_fp8(
                ptr(x), ptr(lw.w), ptr(ops._expert_block_scale(lw)), ptr(y), ptr(self.group_begin),  # pylint: disable=protected-access
                ptr(self.group_count), ptr(self.group_slab), ctypes.c_int(self.e_local), ctypes.c_int(self.e_local),
                ctypes.c_int(rows), ctypes.c_int(hint), ctypes.c_int(n), ctypes.c_int(k), ctypes.c_int(x.stride(0)),
                ctypes.c_int(n), ctypes.c_int(DTYPE_CODE[x.dtype]), ctypes.c_int(DTYPE_CODE[x.dtype]),
                ptr(status_word(x.device)), stream_ptr())
            check(rc, "mlcb_gemm_grouped_fp8")
            return y
        q4 = lw.q4_tileable(k) and x.dtype == lw.scale.dtype
        w = lw.q4_tiles() if q4 else (lw.w if lw.kind == "dense" else lw.dense(x.dtype))
        y = torch.empty(rows, n, dtype=x.dtype, device=x.device)
        rc = lib().mlcb_gemm_grouped_table(
            ptr(x), ptr(w), ptr(w) if q4 else ptr(None), ptr(y), ptr(self.group_begin),
            ptr(self.group_count), ptr(self.group_slab), ctypes.c_int(self.e_local),
            ctypes.c_int(self.e_local), ctypes.c_int(rows), ctypes.c_int(hint), ctypes.c_int(n), ctypes.c_int(k),
            ctypes.c_int(x.stride(0)), ctypes.c_int(n), ctypes.c_int(DTYPE_CODE[x.dtype]),
            ctypes.c_int(DTYPE_CODE[x.dtype]), ptr(status_word(x.device)), stream_ptr())
        check(rc, "mlcb_gemm_grouped_table")
        return y


def expert_parallel_ffn(model, h: torch.Tensor, weights: torch.Tensor, experts: torch.Tensor, w13, w2
                        ) -> torch.Tensor:
    """MoE FFN of all tokens ``h [T, hidden]`` (replicated on the ranks): each rank dispatches its token
    slice through the all-to-all exchange and every rank receives the expert outputs of all tokens."""
    ep: Optional[ExpertParallel] = getattr(model, "ep", None)
    if ep is None:
        raise RuntimeError("expert parallelism was requested but its buffers were not created")
    act = "silu" if model.cfg.hidden_act == "silu" else "gelu"
    return ep.ffn(h, weights, experts, w13, w2, act)
