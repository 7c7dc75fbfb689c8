"""Block-scaled fp8 linear layers (``fp8_e4m3fn_bf16_block_scale``): weights stay fp8 e4m3 in memory
with one fp32 scale per 128 x 128 block and are expanded to the activation dtype inside the tcgen05
GEMM's dequant stage (``gemm_kernel<2>``), so a decode step reads half the bytes of a bf16 model.

Reference: ``quantization/block_scale_quantization.py`` and its CUTLASS / Triton group GEMMs
(``op/cutlass.py:15-160``, ``op/triton.py``).  Activations are kept in 16 bits here (the reference
also quantises them to fp8 per 1 x 128 group); the oracle is the fp32 product with the dequantised
weights.
"""

from __future__ import annotations

from ctypes import c_int
from typing import Optional

import torch

from ._lib import DTYPE_CODE, check, lib, ptr, status_word, stream_ptr


def linear_fp8_block(x: torch.Tensor, lw, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K]`` (fp16 / bf16) times the fp8 weight ``lw.w [N, K]`` with ``lw.scale [N/128, K/128]``."""
    from . import _gemm_scratch  # pylint: disable=import-outside-toplevel

    m, k = x.shape
    n = lw.w.shape[0]
    od = out_dtype or x.dtype
    y = torch.empty(m, n, dtype=od, device=x.device)
    if m == 0:
        return y
    if tuple(lw.quant.block_size) != (128, 128) if lw.quant is not None else False:
        raise ValueError("only 128 x 128 scale blocks are supported")
    x2 = x if x.stride(-1) == 1 else x.contiguous()
    scale = lw.scale if lw.scale.dtype == torch.float32 else lw.scale.float()
    rc = lib().mlcb_gemm_fp8(ptr(x2), ptr(lw.w), ptr(scale.contiguous()), ptr(lw.bias), ptr(y), c_int(m), c_int(n),
                             c_int(k), c_int(x2.stride(0)), c_int(n), c_int(DTYPE_CODE[x.dtype]),
                             c_int(DTYPE_CODE[od]), ptr(status_word(x.device)), *_gemm_scratch(x.device),
                             stream_ptr())
    check(rc, f"mlcb_gemm_fp8(M={m},N={n},K={k})")
    return y
