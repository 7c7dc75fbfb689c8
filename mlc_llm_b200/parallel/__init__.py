"""Multi-GPU plumbing: one process per GPU over ``torch.distributed``.

Rank 0 hosts the serving engine (scheduler, KV manager, sampler host) and broadcasts one packed
descriptor per model step; every other rank runs :func:`worker_loop` and executes the same forward
on its shard.  This replaces the reference's Disco session (controller thread + one worker process
per GPU, ``cpp/serve/engine.cc:772-883``; every model call a broadcast RPC,
``cpp/serve/function_table.cc:53-65``).

Ranks are laid out ``rank = pp_rank * tp_size + tp_rank``: tensor-parallel groups are contiguous,
pipeline stages are strided (reference: workers = shards x stages, ``num_groups = stages``).

Collectives: the baseline tensor-parallel all-reduce is NCCL (``backend="nccl"``; gloo for CPU ranks
in tests).  The fused GEMM+collective kernels live in ``parallel/fused.py`` and use symmetric peer
buffers from ``parallel/symm.py``.
"""

from __future__ import annotations

import datetime
import os
import pickle
import sys
import time
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

_OPS = {"forward": 1, "move": 2, "shutdown": 3, "reset": 4, "forward_async": 5, "forward_part": 6}
_OPS_INV = {v: k for k, v in _OPS.items()}
_DT = {np.dtype(np.int32): 0, np.dtype(np.float32): 1, np.dtype(np.int64): 2}
_DT_INV = {0: np.int32, 1: np.float32, 2: np.int64}
_HEADER_WORDS = 256


def env_world() -> Tuple[int, int, int]:
    """(rank, world_size, local_rank) from the torchrun environment; (0, 1, 0) when absent."""
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)),
            int(os.environ.get("LOCAL_RANK", 0)))


class Communicator:
    """Process-group wrapper with the handful of operations the serving path needs."""

    def __init__(self, tp_size: int, pp_size: int = 1, device: Optional[torch.device] = None,
                 timeout_s: float = 600.0, backend: Optional[str] = None):
        rank, world, local = env_world()
        if tp_size * pp_size != world:
            raise ValueError(f"tp ({tp_size}) x pp ({pp_size}) != world size ({world})")
        self.rank, self.world_size = rank, world
        self.tp_size, self.pp_size = tp_size, pp_size
        self.tp_rank, self.pp_rank = rank % tp_size, rank // tp_size
        if device is None:
            if torch.cuda.is_available():
                torch.cuda.set_device(local)
                device = torch.device("cuda", local)
            else:
                device = torch.device("cpu")
        self.device = device
        if device.type == "cuda":
            torch.cuda.set_device(device)  # object collectives stage through the current device
        backend = backend or ("nccl" if device.type == "cuda" else "gloo")
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            kwargs = {}
            if backend == "nccl":
                kwargs["device_id"] = device
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        self.backend = backend
        # tensor-parallel group of this rank and, per tp_rank, the pipeline chain
        self.tp_group = None
        for s in range(pp_size):
            ranks = list(range(s * tp_size, (s + 1) * tp_size))
            g = dist.new_group(ranks) if (pp_size > 1) else dist.group.WORLD
            if s == self.pp_rank:
                self.tp_group = g
        self.world_group = dist.group.WORLD
        self._header = torch.zeros(_HEADER_WORDS, dtype=torch.int64,
                                   device=device if backend == "nccl" else torch.device("cpu"))
        # Step descriptors travel over a host-side (gloo) group: a worker then receives the next step's
        # descriptor while its GPU still runs the current step, instead of behind it in stream order.
        self.ctl_group = dist.new_group(backend="gloo") if (backend == "nccl" and world > 1) else None
        self._ctl_header = torch.zeros(_HEADER_WORDS, dtype=torch.int64)
        self.fused = None  # parallel.fused.FusedCollectives when enabled
        self.launches = 0

    # ---------------------------------------------------------------- collectives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """In-place sum over the tensor-parallel group."""
        if self.tp_size > 1:
            if self.fused is not None and self.fused.can_all_reduce(x):
                self.fused.all_reduce(x)
            else:
                dist.all_reduce(x, group=self.tp_group)
            self.launches += 1
        return x

    def broadcast_tokens(self, tokens: torch.Tensor) -> None:
        """The tokens rank 0 sampled, to every rank of its tensor-parallel group, device to device
        (they are the next step's inputs and never visit the host on the way). Also carries the feature rows
        of an EAGLE draft call: any tensor whose shape and dtype the ranks agree on."""
        if self.tp_size > 1:
            dist.broadcast(tokens, src=self.pp_rank * self.tp_size, group=self.tp_group)
            self.launches += 1

    # ---------------------------------------------------------------- pipeline stages (NCCL p2p)
    def send_to_next_stage(self, x: torch.Tensor) -> None:
        """Hidden state to the same tensor-parallel rank of the next stage (reference:
        ``runtime.disco.send_to_next_group``, ``compiler_pass/pipeline_parallel_rewrite.py:105-200``).
        NCCL p2p is stream-ordered, so the sender moves on to its next work immediately."""
        dist.send(x.contiguous(), dst=self.rank + self.tp_size)
        self.launches += 1

    def recv_from_prev_stage(self, x: torch.Tensor) -> None:
        dist.recv(x, src=self.rank - self.tp_size)
        self.launches += 1

    def send_logits_to_rank0(self, logits: torch.Tensor) -> None:
        dist.send(logits.contiguous(), dst=0)
        self.launches += 1

    def recv_logits_from_last_stage(self, logits: torch.Tensor) -> None:
        dist.recv(logits, src=(self.pp_size - 1) * self.tp_size)
        self.launches += 1

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier()

    def max_over_ranks(self, value: float) -> float:
        if self.world_size == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=self._header.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def agree_on_capacity(self, res: dict) -> dict:
        """Every rank adopts rank 0's engine configuration / page count, bounded by the minimum
        page count any rank can afford."""
        pages = torch.tensor([int(res["num_pages"])], dtype=torch.int64, device=self._header.device)
        dist.all_reduce(pages, op=dist.ReduceOp.MIN)
        box = [res if self.rank == 0 else None]
        dist.broadcast_object_list(box, src=0, device=self._header.device)
        out = dict(box[0])
        out["num_pages"] = int(pages.item())
        return out

    # ---------------------------------------------------------------- step broadcast
    def broadcast_step(self, op: str, model_id: int, arrays: Dict[str, np.ndarray], meta: dict) -> None:
        """Rank 0: ship a packed step descriptor to every other rank."""
        if self.world_size == 1:
            return
        names = list(arrays)
        if 4 + 3 * len(names) > _HEADER_WORDS:
            raise ValueError("too many arrays in one step descriptor")
        words = 0
        hdr = [_OPS[op], model_id, len(names), 0]
        for n in names:
            a = arrays[n]
            w = a.size * (2 if a.dtype.itemsize == 8 else 1)
            hdr += [_NAME_ID[n], _DT[a.dtype], a.size]
            words += (w + 3) & ~3
        hdr[3] = words
        h = torch.tensor(hdr + [0] * (_HEADER_WORDS - len(hdr)), dtype=torch.int64)
        host_side = self.ctl_group is not None or self.backend != "nccl"
        if host_side:
            self._ctl_header.copy_(h)
            dist.broadcast(self._ctl_header, src=0, group=self.ctl_group)
        else:
            self._header.copy_(h)
            dist.broadcast(self._header, src=0)
        if words:
            buf = np.zeros(words, dtype=np.int32)
            off = 0
            for n in names:
                a = arrays[n]
                w = a.size * (2 if a.dtype.itemsize == 8 else 1)
                if w:
                    buf[off:off + w] = a.reshape(-1).view(np.int32)
                off += (w + 3) & ~3
            t = torch.from_numpy(buf)
            if host_side:
                dist.broadcast(t, src=0, group=self.ctl_group)
            else:
                t = t.to(self.device, non_blocking=True)
                dist.broadcast(t, src=0)

    def receive_step(self):
        """Ranks > 0: block for the next descriptor. Returns (op, model_id, arrays)."""
        host_side = self.ctl_group is not None or self.backend != "nccl"
        if host_side:
            dist.broadcast(self._ctl_header, src=0, group=self.ctl_group)
            hdr = self._ctl_header.tolist()
        else:
            dist.broadcast(self._header, src=0)
            hdr = self._header.cpu().tolist()
        op, model_id, count, words = _OPS_INV[hdr[0]], hdr[1], hdr[2], hdr[3]
        arrays: Dict[str, np.ndarray] = {}
        if words:
            if host_side:
                t = torch.empty(words, dtype=torch.int32)
                dist.broadcast(t, src=0, group=self.ctl_group)
            else:
                t = torch.empty(words, dtype=torch.int32, device=self.device)
                dist.broadcast(t, src=0)
            buf = t.cpu().numpy()
        else:
            buf = np.zeros(0, dtype=np.int32)
        off = 0
        for i in range(count):
            nid, dt, size = hdr[4 + 3 * i: 7 + 3 * i]
            npdt = _DT_INV[dt]
            w = size * (2 if npdt == np.int64 else 1)
            arrays[_ID_NAME[nid]] = buf[off:off + w].view(npdt).copy()
            off += (w + 3) & ~3
        return op, model_id, arrays

    def shutdown_workers(self) -> None:
        if self.world_size > 1 and self.rank == 0:
            self.broadcast_step("shutdown", 0, {}, {})

    def destroy(self) -> None:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # pylint: disable=broad-except
                pass


_ARRAY_NAMES = ["token_ids", "positions", "slots", "q_seq", "q_kvlen", "q_kvstart", "page_indptr",
                "page_indices", "page_copies", "q_indptr", "seq_lens", "append_lens", "tree_mask", "moves",
                "s_logit_token_index", "s_top_k", "s_pen_row", "s_pen_token", "s_pen_count", "s_bias_row",
                "s_bias_token", "s_mask_rows", "s_mask_bits", "s_prob_slots", "s_temperature", "s_top_p",
                "s_uniform", "s_penalties", "s_bias_value", "tile_seq", "tile_qstart", "tile_ntok", "dec_seq", "dec_qstart",
                "dec_ntok", "token_src", "seq_ids", "seq_forks"]
_NAME_ID = {n: i for i, n in enumerate(_ARRAY_NAMES)}
_ID_NAME = dict(enumerate(_ARRAY_NAMES))


def worker_loop(executor, comm: Communicator) -> None:
    """Body of every rank other than 0: mirror rank 0's model calls until told to stop."""
    report = os.environ.get("MLCB_STEP_TIMES") == "1"
    recv_s = step_s = 0.0
    steps = 0
    while True:
        t0 = time.perf_counter()
        op, model_id, arrays = comm.receive_step()
        t1 = time.perf_counter()
        if op == "shutdown":
            if report and steps:
                print(f"[rank {comm.rank}] {steps} steps: receive {recv_s * 1e3 / steps:.3f} ms/step, "
                      f"launch {step_s * 1e3 / steps:.3f} ms/step", file=sys.stderr, flush=True)
            return
        if op == "reset":
            executor.reset()
            continue
        executor.worker_step(op, model_id, arrays, None)
        recv_s += t1 - t0
        step_s += time.perf_counter() - t1
        steps += 1
