"""Host side of the tensor-core paged attention kernel: query tiling and the launch wrapper."""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Dict, Optional

import numpy as np
import torch

from ._lib import DTYPE_CODE, check, lib, ptr, status_word, stream_ptr


def build_tiles(q_indptr: np.ndarray, group: int) -> Dict[str, np.ndarray]:
    """Split every sequence's appended tokens into tiles of ``128 // group`` tokens.

    Returns int32 arrays ``tile_seq`` (batch slot), ``tile_qstart`` (first global token index) and
    ``tile_ntok``. Decode (one token per sequence) yields one tile per sequence.
    """
    tpt = max(1, 128 // group)
    q_indptr = np.asarray(q_indptr, dtype=np.int64)
    lens = np.diff(q_indptr)
    ntiles = (lens + tpt - 1) // tpt
    total = int(ntiles.sum())
    seq = np.repeat(np.arange(len(lens), dtype=np.int64), ntiles)
    first_tile = np.concatenate(([0], np.cumsum(ntiles)[:-1]))
    local = np.arange(total, dtype=np.int64) - np.repeat(first_tile, ntiles)
    qstart = q_indptr[seq] + local * tpt
    ntok = np.minimum(tpt, q_indptr[seq + 1] - qstart)
    return {"tile_seq": seq.astype(np.int32), "tile_qstart": qstart.astype(np.int32),
            "tile_ntok": ntok.astype(np.int32)}


@dataclasses.dataclass
class AttentionPlan:
    """Device-resident tiling of one forward call (shared by all layers)."""

    tile_seq: torch.Tensor
    tile_qstart: torch.Tensor
    tile_ntok: torch.Tensor
    q_kvlen: torch.Tensor
    page_indptr: torch.Tensor
    page_indices: torch.Tensor
    num_tiles: int
    use_tensor_core: bool = True


def attention_tcgen05(q: torch.Tensor, kv_pages: torch.Tensor, out: torch.Tensor,
                      lse: Optional[torch.Tensor], plan: AttentionPlan, hq: int, hkv: int,
                      sm_scale: float) -> None:
    """``q``: [T, hq*128] view (row stride may be larger); ``kv_pages``: one layer's cache."""
    rc = lib().mlcb_attn_tc(ptr(q), ptr(kv_pages), ptr(out), ptr(lse), ptr(plan.tile_seq),
                            ptr(plan.tile_qstart), ptr(plan.tile_ntok), ptr(plan.q_kvlen),
                            ptr(plan.page_indptr), ptr(plan.page_indices), ctypes.c_int(plan.num_tiles),
                            ctypes.c_longlong(q.stride(0)), ctypes.c_int(hq), ctypes.c_int(hkv),
                            ctypes.c_longlong(kv_pages.shape[0]), ctypes.c_float(sm_scale),
                            ctypes.c_int(DTYPE_CODE[q.dtype]), ptr(status_word(q.device)), stream_ptr())
    check(rc, "mlcb_attn_tc")
