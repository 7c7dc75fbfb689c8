"""Host side of the tensor-core paged attention kernel: query tiling and the launch wrapper."""

from __future__ import annotations

import ctypes
import dataclasses
from typing import Dict, Optional

import numpy as np
import torch

from ._lib import DTYPE_CODE, check, lib, ptr, status_word, stream_ptr


def build_tiles(q_indptr: np.ndarray, group: int, decode_items: bool = True) -> Dict[str, np.ndarray]:
    """Split the appended tokens of a batch into work items for the two attention kernels.

    Sequences whose chunk fits 16 query rows (``tokens * group <= 16``: decode and short verify
    chunks) become one item each for the decode kernel (``dec_seq``, ``dec_qstart``, ``dec_ntok``).
    The others are cut into tiles of ``128 // group`` tokens for the tcgen05 kernel (``tile_seq``,
    ``tile_qstart``, ``tile_ntok``). All arrays are int32; ``*_qstart`` are global token indices.
    ``decode_items=False`` sends every sequence to the tcgen05 kernel.
    """
    tpt = max(1, 128 // group)
    q_indptr = np.asarray(q_indptr, dtype=np.int64)
    lens_all = np.diff(q_indptr)
    small = (lens_all * group <= 16) & (lens_all > 0) if group <= 16 and decode_items \
        else np.zeros(len(lens_all), bool)
    dec_idx = np.nonzero(small)[0]
    out = {"dec_seq": dec_idx.astype(np.int32), "dec_qstart": q_indptr[dec_idx].astype(np.int32),
           "dec_ntok": lens_all[dec_idx].astype(np.int32)}
    lens = np.where(small, 0, lens_all)
    ntiles = (lens + tpt - 1) // tpt
    total = int(ntiles.sum())
    seq = np.repeat(np.arange(len(lens), dtype=np.int64), ntiles)
    first_tile = np.concatenate(([0], np.cumsum(ntiles)[:-1]))
    local = np.arange(total, dtype=np.int64) - np.repeat(first_tile, ntiles)
    qstart = q_indptr[seq] + local * tpt
    ntok = np.minimum(tpt, q_indptr[seq + 1] - qstart)
    out.update({"tile_seq": seq.astype(np.int32), "tile_qstart": qstart.astype(np.int32),
                "tile_ntok": ntok.astype(np.int32)})
    return out


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
    dec_seq: Optional[torch.Tensor] = None
    dec_qstart: Optional[torch.Tensor] = None
    dec_ntok: Optional[torch.Tensor] = None
    num_dec: int = 0
    dec_splits: int = 1
    max_pages: int = 0


def attention_tcgen05(q: torch.Tensor, kv_pages: torch.Tensor, out: torch.Tensor,
                      lse: Optional[torch.Tensor], plan: AttentionPlan, hq: int, hkv: int,
                      sm_scale: float, q_kvstart: Optional[torch.Tensor] = None, sink: int = 0,
                      tree_mask: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """``q``: [T, hq*128] view (row stride may be larger); ``kv_pages``: one layer's cache.
    ``q_kvstart`` (+ ``sink``), ``tree_mask`` and ``softcap`` select the kernel's masked variant."""
    rc = lib().mlcb_attn_tc(ptr(q), ptr(kv_pages), ptr(out), ptr(lse), ptr(plan.tile_seq),
                            ptr(plan.tile_qstart), ptr(plan.tile_ntok), ptr(plan.q_kvlen),
                            ptr(plan.page_indptr), ptr(plan.page_indices), ctypes.c_int(plan.num_tiles),
                            ctypes.c_longlong(q.stride(0)), ctypes.c_int(hq), ctypes.c_int(hkv),
                            ctypes.c_longlong(kv_pages.shape[0]), ctypes.c_float(sm_scale),
                            ctypes.c_int(DTYPE_CODE[q.dtype]), ptr(status_word(q.device)), stream_ptr(),
                            ptr(q_kvstart), ptr(tree_mask), ctypes.c_int(int(sink)), ctypes.c_float(float(softcap)))
    check(rc, "mlcb_attn_tc")


_SM_COUNT = {}


def choose_splits(num_items: int, hkv: int, max_pages: int, device: torch.device) -> int:
    """Split the KV range when (items x kv heads) alone cannot fill the GPU (few long sequences)."""
    key = device.index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    ctas = num_items * hkv
    target = 2 * _SM_COUNT[key]  # the decode kernel keeps two persistent CTAs per SM
    if ctas >= target or max_pages < 16:
        return 1
    return int(max(1, min(32, target // max(1, ctas), max_pages // 8)))


def attention_decode(q: torch.Tensor, kv_pages: torch.Tensor, out: torch.Tensor,
                     lse: Optional[torch.Tensor], plan: AttentionPlan, hq: int, hkv: int,
                     sm_scale: float, q_kvstart: Optional[torch.Tensor] = None, sink: int = 0,
                     tree_mask: Optional[torch.Tensor] = None, softcap: float = 0.0) -> None:
    """Decode-kernel launch for the items of ``plan`` with at most 16 query rows each; the mask arguments
    select its masked variant (same rule as :func:`attention_tcgen05`)."""
    splits = plan.dec_splits
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty(plan.num_dec * hkv * splits * 16 * 128, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(plan.num_dec * hkv * splits * 16 * 2, dtype=torch.float32, device=q.device)
    rc = lib().mlcb_attn_decode(ptr(q), ptr(kv_pages), ptr(out), ptr(lse), ptr(plan.dec_seq),
                                ptr(plan.dec_qstart), ptr(plan.dec_ntok), ptr(plan.q_kvlen),
                                ptr(plan.page_indptr), ptr(plan.page_indices), ctypes.c_int(plan.num_dec),
                                ctypes.c_longlong(q.stride(0)), ctypes.c_int(hq), ctypes.c_int(hkv),
                                ctypes.c_longlong(kv_pages.shape[0]), ctypes.c_float(sm_scale),
                                ctypes.c_int(DTYPE_CODE[q.dtype]), ctypes.c_int(splits), ptr(part_o),
                                ptr(part_ml), ptr(status_word(q.device)), stream_ptr(), ptr(q_kvstart),
                                ptr(tree_mask), ctypes.c_int(int(sink)), ctypes.c_float(float(softcap)))
    check(rc, "mlcb_attn_decode")
