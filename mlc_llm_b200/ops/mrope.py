"""Multimodal rotary positions (Qwen2.5-VL): every token carries a (time, height, width) position
triple; text tokens use the same number on all three axes, the tokens of an image or video grid count
along their own axes, and the rotary frequency bands of a head are split between the axes.

Reference: ``python/mlc_llm/op/mrope.py`` (``get_mrope_position_ids``, ``apply_multimodal_rotary_pos_emb``,
``VisionPositionMetadata``).  For text-only prompts the three axes agree and the rotation equals plain
rotary embedding, which is what the serving path runs; this module is the host-side position builder and
the reference rotation for prompts with vision grids.
"""

from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclasses.dataclass
class VisionPositionMetadata:
    """Token ids and grid constants needed to lay out vision tokens."""

    vision_start_token_id: int
    image_token_id: int
    video_token_id: int
    spatial_merge_size: int = 2
    tokens_per_second: float = 2.0


def _grid_positions(t: int, h: int, w: int, offset: int, time_step: float) -> np.ndarray:
    tt = (np.arange(t, dtype=np.float32) * time_step).astype(np.int64)
    axes = np.stack([np.repeat(tt, h * w),
                     np.tile(np.repeat(np.arange(h, dtype=np.int64), w), t),
                     np.tile(np.arange(w, dtype=np.int64), t * h)])
    return axes + offset


def sequence_position_ids(tokens: Sequence[int], meta: VisionPositionMetadata,
                          image_grids: Sequence[Sequence[int]] = (), video_grids: Sequence[Sequence[int]] = (),
                          second_per_grid: Optional[Sequence[float]] = None) -> Tuple[np.ndarray, int]:
    """Positions ``[3, T]`` of one prompt and the offset ``delta`` a later decode step adds to its
    token index (``position = index + delta``).

    A vision block is announced by ``vision_start_token_id`` followed by the image / video placeholder;
    the block's grid ``(t, h, w)`` is given in patches and shrinks by ``spatial_merge_size`` on h and w.
    Text before a block continues from the largest position used so far plus one; so does whatever
    follows the block.
    """
    toks = np.asarray(tokens, dtype=np.int64)
    n = len(toks)
    chunks: List[np.ndarray] = []
    next_pos = 0
    i = 0
    img_i = vid_i = 0
    m = meta.spatial_merge_size
    starts = np.nonzero(toks[:-1] == meta.vision_start_token_id)[0] if n > 1 else []
    for s in starts:
        kind = int(toks[s + 1])
        if kind not in (meta.image_token_id, meta.video_token_id) or s + 1 < i:
            continue
        if kind == meta.image_token_id:
            if img_i >= len(image_grids):
                raise ValueError("more image blocks in the prompt than image grids")
            t, h, w = (int(x) for x in image_grids[img_i])
            img_i += 1
            step = 0.0
        else:
            if vid_i >= len(video_grids):
                raise ValueError("more video blocks in the prompt than video grids")
            t, h, w = (int(x) for x in video_grids[vid_i])
            spg = 1.0 if second_per_grid is None else float(second_per_grid[vid_i])
            vid_i += 1
            step = spg * meta.tokens_per_second
        if h % m or w % m:
            raise ValueError(f"grid {h}x{w} is not divisible by the spatial merge size {m}")
        h, w = h // m, w // m
        text_len = s + 1 - i  # text up to and including the start marker
        chunks.append(np.broadcast_to(np.arange(text_len, dtype=np.int64) + next_pos, (3, text_len)))
        next_pos += text_len
        grid = _grid_positions(t, h, w, next_pos, step)
        chunks.append(grid)
        next_pos = int(grid.max()) + 1
        i = s + 1 + t * h * w
    if i < n:
        chunks.append(np.broadcast_to(np.arange(n - i, dtype=np.int64) + next_pos, (3, n - i)))
        next_pos += n - i
    if not chunks:
        return np.zeros((3, 0), dtype=np.int64), 0
    pos = np.concatenate(chunks, axis=1)
    if pos.shape[1] != n:
        raise ValueError("vision grids do not match the number of placeholder tokens in the prompt")
    return pos, int(pos.max()) + 1 - n


def mrope_position_ids(input_ids: np.ndarray, meta: VisionPositionMetadata,
                       attention_mask: Optional[np.ndarray] = None, image_grids: Sequence[Sequence[int]] = (),
                       video_grids: Sequence[Sequence[int]] = (), second_per_grid: Optional[Sequence[float]] = None
                       ) -> Tuple[np.ndarray, np.ndarray]:
    """Batch form: ``input_ids [B, T]`` (padded; ``attention_mask`` marks real tokens) -> positions
    ``[3, B, T]`` (padding gets 1) and per-row deltas ``[B, 1]``. Grids are consumed in row order."""
    ids = np.asarray(input_ids, dtype=np.int64)
    b, t = ids.shape
    out = np.ones((3, b, t), dtype=np.int64)
    deltas = np.zeros((b, 1), dtype=np.int64)
    img_i = vid_i = 0
    for r in range(b):
        keep = np.ones(t, dtype=bool) if attention_mask is None else np.asarray(attention_mask[r]).astype(bool)
        row = ids[r][keep]
        starts = np.nonzero(row[:-1] == meta.vision_start_token_id)[0] if len(row) > 1 else []
        n_img = int(sum(row[s + 1] == meta.image_token_id for s in starts))
        n_vid = int(sum(row[s + 1] == meta.video_token_id for s in starts))
        spg = None if second_per_grid is None else list(second_per_grid[vid_i: vid_i + n_vid])
        pos, delta = sequence_position_ids(row.tolist(), meta, list(image_grids[img_i: img_i + n_img]),
                                           list(video_grids[vid_i: vid_i + n_vid]), spg)
        img_i, vid_i = img_i + n_img, vid_i + n_vid
        out[:, r, keep] = pos
        deltas[r, 0] = delta
    return out, deltas


def apply_mrope(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                mrope_section: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotate ``q [T, Hq, D]`` and ``k [T, Hk, D]`` (half-split pairs) with positions ``[3, T]``:
    frequency band ``j`` of a head takes its angle from the axis that owns it, the bands being dealt to
    (time, height, width) in runs of ``mrope_section`` entries."""
    if sum(mrope_section) != inv_freq.numel():
        raise ValueError(f"mrope_section {list(mrope_section)} must add up to {inv_freq.numel()} frequency bands")
    owner = torch.repeat_interleave(torch.arange(3), torch.as_tensor(list(mrope_section))).to(inv_freq.device)
    angles = positions.to(inv_freq.device).float().unsqueeze(-1) * inv_freq.float()      # [3, T, D/2]
    angle = angles.gather(0, owner.view(1, 1, -1).expand(1, angles.shape[1], -1))[0]     # [T, D/2]
    cos = torch.cat([angle.cos(), angle.cos()], dim=-1).unsqueeze(1)
    sin = torch.cat([angle.sin(), angle.sin()], dim=-1).unsqueeze(1)

    def rot(x: torch.Tensor) -> torch.Tensor:
        half = x.shape[-1] // 2
        xf = x.float()
        return (xf * cos + torch.cat([-xf[..., half:], xf[..., :half]], dim=-1) * sin).to(x.dtype)

    return rot(q), rot(k)
