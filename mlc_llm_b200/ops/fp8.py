"""Block-scaled fp8 linear layers (``fp8_e4m3fn_bf16_block_scale``): weights stay fp8 e4m3 in memory
with one fp32 scale per 128 x 128 block.

Two kernels serve them.  W8A8 (the default from 17 tokens up, when K is a multiple of 128): the activations
are quantised on the fly to e4m3 with one scale per row and 128-element group (``mlcb_act_quant_fp8``) and
both operands reach the tensor core as fp8 (``gemm_fp8.cu``, ``tcgen05.mma kind::f8f6f4``, group-wise
promotion of the partial sums) -- the reference's scheme (``quantization/block_scale_quantization.py:603-700``,
``op/cutlass.py:138-279``).  W8A16 (``MLCB_FP8_ACT=0``, small batches, odd K): the weights are expanded to
the activation dtype inside the 16-bit GEMM's dequant stage (``gemm_kernel<2>``).
"""

from __future__ import annotations

import os
from ctypes import c_int, c_longlong
from typing import Optional, Tuple

import torch

from ._lib import DTYPE_CODE, check, lib, ptr, status_word, stream_ptr


_FP8_ACT = os.environ.get("MLCB_FP8_ACT", "1") != "0"
_W8A8_MIN_TOKENS = 17


def act_quant_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [M, K]`` (fp16 / bf16) -> (e4m3 ``[M, K]``, fp32 scales ``[K / 128, ld]``, transposed, one per row
    and 128-element group: ``max(|x|, 1e-10) / 448``).  ``ld`` >= M leaves room for the last token tile."""
    m, k = x.shape
    # the GEMM reads one contiguous run of scales per token tile (up to 256 tokens, tile count x tile width
    # can exceed M by a sixteenth): leave that room
    ld = (m + m // 16 + 256 + 127) // 128 * 128
    xq = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=x.device)
    scale_t = torch.zeros((k + 127) // 128, ld, dtype=torch.float32, device=x.device)
    x2 = x if x.stride(-1) == 1 else x.contiguous()
    rc = lib().mlcb_act_quant_fp8(ptr(x2), ptr(xq), ptr(scale_t), c_int(m), c_int(k), c_longlong(x2.stride(0)),
                                  c_int(ld), c_int(DTYPE_CODE[x.dtype]), stream_ptr())
    check(rc, f"mlcb_act_quant_fp8(M={m},K={k})")
    return xq, scale_t


def linear_fp8_w8a8(x: torch.Tensor, lw, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """fp8 x fp8 product with on-the-fly activation quantisation; ``K`` must be a multiple of 128."""
    m, k = x.shape
    n = lw.w.shape[0]
    od = out_dtype or x.dtype
    y = torch.empty(m, n, dtype=od, device=x.device)
    if m == 0:
        return y
    xq, xs = act_quant_fp8(x)
    scale = lw.block_scale()
    rc = lib().mlcb_gemm_fp8_w8a8(ptr(xq), ptr(xs), ptr(lw.w), ptr(scale), ptr(lw.bias), ptr(y), c_int(m),
                                  c_int(n), c_int(k), c_int(n), c_int(xs.shape[1]), c_int(DTYPE_CODE[od]),
                                  ptr(status_word(x.device)), stream_ptr())
    check(rc, f"mlcb_gemm_fp8_w8a8(M={m},N={n},K={k})")
    return y


def linear_fp8_block(x: torch.Tensor, lw, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K]`` (fp16 / bf16) times the fp8 weight ``lw.w [N, K]`` with ``lw.scale [N/128, K/128]``."""
    from . import _gemm_scratch  # pylint: disable=import-outside-toplevel

    m, k = x.shape
    n = lw.w.shape[0]
    od = out_dtype or x.dtype
    if lw.kind == "fp8_block" and lw.quant is not None and tuple(lw.quant.block_size) != (128, 128):
        raise ValueError("only 128 x 128 scale blocks are supported")
    if _FP8_ACT and m >= _W8A8_MIN_TOKENS and k % 128 == 0 and od in (torch.float16, torch.bfloat16) \
            and (lw.bias is None or lw.bias.dtype == od):
        return linear_fp8_w8a8(x, lw, od)
    y = torch.empty(m, n, dtype=od, device=x.device)
    if m == 0:
        return y
    x2 = x if x.stride(-1) == 1 else x.contiguous()
    scale = lw.block_scale()
    rc = lib().mlcb_gemm_fp8(ptr(x2), ptr(lw.w), ptr(scale), ptr(lw.bias), ptr(y), c_int(m), c_int(n),
                             c_int(k), c_int(x2.stride(0)), c_int(n), c_int(DTYPE_CODE[x.dtype]),
                             c_int(DTYPE_CODE[od]), ptr(status_word(x.device)), *_gemm_scratch(x.device),
                             stream_ptr())
    check(rc, f"mlcb_gemm_fp8(M={m},N={n},K={k})")
    return y
