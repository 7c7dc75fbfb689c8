"""Quantization schemes: registry plus bit-exact pack / unpack in PyTorch.

The on-disk layouts are those of the reference (``python/mlc_llm/quantization/quantization.py:31-201``):

* group quantization ``q{3,4}{f16,bf16,f32}_{0,1,2}`` -- ``group_quantization.py:235-306`` and the bit
  packing of ``quantization/utils.py:136-188``: for a weight ``[N, K]``, ``scale = max|w| / max_int``
  per group of ``group_size`` along K, ``q = clamp(round(w / scale + max_int), 0, 2 * max_int)``,
  element ``j`` of a storage word at bits ``bits * (j % elems_per_word)``;
* ``fp8_e4m3fn_bf16_block_scale`` -- ``block_scale_quantization.py:198-205``: ``weight`` e4m3 plus
  ``weight_scale_inv [ceil(N/128), ceil(K/128)]`` fp32; activations are quantised per row per
  128-wide group at run time;
* ``e4m3_e4m3_f16`` / ``e5m2_e5m2_f16`` -- ``per_tensor_quantization.py:30-140``: fp8 weight plus a
  scalar fp32 scale.

The GPU-resident int4 layout differs from the artifact layout by a fixed nibble permutation inside
each 32-bit word (see :func:`to_device_layout_q4`) so that the GEMM's dequant warps produce two
consecutive fp16 values per bit operation.
"""

from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Tuple

import torch

_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclasses.dataclass(frozen=True)
class Quantization:
    """Description of one named quantization mode."""

    name: str
    kind: str  # "no-quant" | "group-quant" | "fp8-per-tensor" | "fp8-block-scale" | "awq" | "ft-quant"
    model_dtype: str
    bits: int = 16
    group_size: int = 0
    storage_dtype: str = "uint32"
    linear_weight_layout: str = "NK"
    quantize_embedding: bool = True
    quantize_final_fc: bool = True
    weight_dtype: str = ""  # fp8 kinds
    activation_dtype: str = ""
    block_size: Tuple[int, int] = (128, 128)
    calibration: str = ""
    static_activation: bool = False

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.model_dtype]

    @property
    def max_int(self) -> int:
        return (1 << (self.bits - 1)) - 1

    @property
    def elems_per_word(self) -> int:
        return 32 // self.bits

    @property
    def words_per_group(self) -> int:
        return (self.group_size + self.elems_per_word - 1) // self.elems_per_word


def _group(name: str, bits: int, dtype: str, group: int, layout: str = "NK", qe=True, qf=True):
    return Quantization(name, "group-quant", dtype, bits=bits, group_size=group,
                        linear_weight_layout=layout, quantize_embedding=qe, quantize_final_fc=qf)


QUANTIZATION: Dict[str, Quantization] = {
    "q0f16": Quantization("q0f16", "no-quant", "float16"),
    "q0bf16": Quantization("q0bf16", "no-quant", "bfloat16"),
    "q0f32": Quantization("q0f32", "no-quant", "float32"),
    "q3f16_0": _group("q3f16_0", 3, "float16", 40, "KN"),
    "q3f16_1": _group("q3f16_1", 3, "float16", 40),
    "q4f16_0": _group("q4f16_0", 4, "float16", 32, "KN"),
    "q4f16_1": _group("q4f16_1", 4, "float16", 32),
    "q4bf16_0": _group("q4bf16_0", 4, "bfloat16", 32, "KN"),
    "q4bf16_1": _group("q4bf16_1", 4, "bfloat16", 32),
    "q4f32_1": _group("q4f32_1", 4, "float32", 32),
    "q4f16_2": _group("q4f16_2", 4, "float16", 32, "NK", qe=False, qf=False),
    # AWQ checkpoints (qweight / qzeros / scales triples) are expanded to 16-bit weights when they are read
    # (loader/huggingface_loader.py), so at run time this is a 16-bit model
    "q4f16_autoawq": Quantization("q4f16_autoawq", "no-quant", "float16"),
    "e5m2_e5m2_f16": Quantization("e5m2_e5m2_f16", "fp8-per-tensor", "float16", bits=8,
                                  weight_dtype="float8_e5m2", activation_dtype="float8_e5m2"),
    "e4m3_e4m3_f16": Quantization("e4m3_e4m3_f16", "fp8-per-tensor", "float16", bits=8,
                                  weight_dtype="float8_e4m3fn", activation_dtype="float8_e4m3fn",
                                  calibration="inference"),
    "e4m3_e4m3_f16_max_calibrate": Quantization(
        "e4m3_e4m3_f16_max_calibrate", "fp8-per-tensor", "float16", bits=8,
        weight_dtype="float8_e4m3fn", activation_dtype="float8_e4m3fn", calibration="max"),
    "fp8_e4m3fn_bf16_block_scale": Quantization(
        "fp8_e4m3fn_bf16_block_scale", "fp8-block-scale", "bfloat16", bits=8,
        weight_dtype="float8_e4m3fn", quantize_embedding=False, quantize_final_fc=False),
    "fp8_e4m3fn_bf16_block_scale_static_activation": Quantization(
        "fp8_e4m3fn_bf16_block_scale_static_activation", "fp8-block-scale", "bfloat16", bits=8,
        weight_dtype="float8_e4m3fn", quantize_embedding=False, quantize_final_fc=False,
        static_activation=True),
}


def get(name: str) -> Quantization:
    if name == "q4f16_ft":
        raise ValueError("q4f16_ft stores weights in the pre-shuffled layout of FasterTransformer's mixed-input "
                         "CUTLASS GEMM, which this build has no kernel for; use q4f16_1 (the same 4-bit group "
                         "quantisation, tensor-core kernel included)")
    if name not in QUANTIZATION:
        raise ValueError(f"unknown quantization {name!r}; known: {sorted(QUANTIZATION)}")
    return QUANTIZATION[name]


# ----------------------------------------------------------------------------- group quantization
def group_quantize(w: torch.Tensor, q: Quantization) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise ``w[..., N, K]`` along K. Returns ``(q_weight [..., N, words] int32-viewed-uint32,
    q_scale [..., N, groups])`` in the artifact layout. Arithmetic is carried out in the model
    dtype exactly as the reference does (scale and the rounded quotient are model-dtype values)."""
    assert q.kind == "group-quant"
    dt = q.torch_dtype
    w = w.to(dt)
    *lead, n, k = w.shape
    g = q.group_size
    ng = (k + g - 1) // g
    pad = ng * g - k
    wp = torch.nn.functional.pad(w, (0, pad)) if pad else w
    wg = wp.reshape(*lead, n, ng, g)
    # max-abs over the valid part of each group (padding contributes 0 <= any abs value)
    max_abs = wg.abs().amax(dim=-1)
    scale = (max_abs.to(dt) / q.max_int).to(dt)
    quot = (wg / scale.unsqueeze(-1)).to(dt) + q.max_int
    qv = torch.clamp(torch.round(quot.to(torch.float32)), 0, 2 * q.max_int)
    qv = torch.nan_to_num(qv, nan=float(q.max_int))  # all-zero group: 0/0 -> centre value
    qv = qv.to(torch.int64).reshape(*lead, n, ng * g)
    epw = q.elems_per_word
    nwords = ng * q.words_per_group
    # pack per group: a group occupies words_per_group words (q3: 40 elems -> 4 words of 10)
    qv = qv.reshape(*lead, n, ng, g)
    padw = q.words_per_group * epw - g
    if padw:
        qv = torch.nn.functional.pad(qv, (0, padw))
    qv = qv.reshape(*lead, n, nwords, epw)
    shifts = (torch.arange(epw, dtype=torch.int64, device=w.device) * q.bits)
    packed = (qv << shifts).sum(dim=-1)
    packed = packed.to(torch.int64)
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    return packed, scale


def group_dequantize(qw: torch.Tensor, qs: torch.Tensor, q: Quantization, k: Optional[int] = None,
                     out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Inverse of :func:`group_quantize` (``(nibble - max_int) * scale``), artifact layout in."""
    epw = q.elems_per_word
    *lead, n, nwords = qw.shape
    ng = qs.shape[-1]
    words = qw.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(epw, dtype=torch.int64, device=qw.device) * q.bits)
    vals = (words.unsqueeze(-1) >> shifts) & ((1 << q.bits) - 1)  # [..., n, nwords, epw]
    vals = vals.reshape(*lead, n, ng, q.words_per_group * epw)[..., : q.group_size]
    dt = out_dtype or q.torch_dtype
    deq = (vals.to(torch.float32) - q.max_int).to(dt) * qs.to(dt).unsqueeze(-1)
    deq = deq.reshape(*lead, n, ng * q.group_size)
    if k is not None and k != deq.shape[-1]:
        deq = deq[..., :k].contiguous()  # kernels read the result through a raw pointer with row stride k
    return deq


def to_device_layout_q4(qw: torch.Tensor) -> torch.Tensor:
    """Permute nibbles inside every 32-bit word from artifact order (nibble j at bits 4j) to the
    GPU-resident order: pair (2j, 2j+1) at bits [4j, 4j+4) and [16+4j, 20+4j). One mask + shift then
    isolates two consecutive weights in the two fp16 halves of a register."""
    x = qw.to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(x)
    for j in range(4):
        lo = (x >> (4 * (2 * j))) & 0xF
        hi = (x >> (4 * (2 * j + 1))) & 0xF
        out |= (lo << (4 * j)) | (hi << (16 + 4 * j))
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def from_device_layout_q4(qw: torch.Tensor) -> torch.Tensor:
    x = qw.to(torch.int64) & 0xFFFFFFFF
    out = torch.zeros_like(x)
    for j in range(4):
        lo = (x >> (4 * j)) & 0xF
        hi = (x >> (16 + 4 * j)) & 0xF
        out |= (lo << (4 * (2 * j))) | (hi << (4 * (2 * j + 1)))
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


# ----------------------------------------------------------------------------- AWQ checkpoints
# AutoAWQ "GEMM" layout (reference: quantization/awq_quantization.py:133-176, quantization/utils.py:15-48):
# qweight [K, N/8] and qzeros [K/g, N/8] pack eight 4-bit values per 32-bit word with output column j of a
# word at nibble (j % 2) * 4 + j // 2; scales [K/g, N]; W[n, k] = (q[k, n] - z[k / g, n]) * s[k / g, n].
_AWQ_NIBBLE = [(j % 2) * 4 + j // 2 for j in range(8)]


def _awq_unpack(words: torch.Tensor) -> torch.Tensor:
    """``[R, C/8]`` int32 -> ``[R, C]`` values 0..15."""
    x = words.to(torch.int64) & 0xFFFFFFFF
    cols = [(x >> (4 * _AWQ_NIBBLE[j])) & 0xF for j in range(8)]
    return torch.stack(cols, dim=-1).reshape(words.shape[0], words.shape[1] * 8)


def awq_pack(values: torch.Tensor) -> torch.Tensor:
    """Inverse of the unpacking above (``[R, C]`` values 0..15 -> ``[R, C/8]`` int32); used to write AWQ-format
    tensors and in tests."""
    r, c = values.shape
    v = values.to(torch.int64).reshape(r, c // 8, 8)
    out = torch.zeros(r, c // 8, dtype=torch.int64)
    for j in range(8):
        out |= (v[..., j] & 0xF) << (4 * _AWQ_NIBBLE[j])
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def awq_dequantize(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                   out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """AWQ tensors of one linear layer -> the dense weight ``[N, K]``.  The group size follows from the
    shapes (``K / scales.shape[0]``)."""
    k, n = qweight.shape[0], qweight.shape[1] * 8
    groups = scales.shape[0]
    if k % groups or scales.shape[1] != n or qzeros.shape[0] != groups:
        raise ValueError("inconsistent AWQ tensor shapes")
    g = k // groups
    q = _awq_unpack(qweight).float()                                   # [K, N]
    z = _awq_unpack(qzeros)[:, :n].float().repeat_interleave(g, dim=0)  # [K, N]
    s = scales.float().repeat_interleave(g, dim=0)
    return ((q - z) * s).t().contiguous().to(out_dtype)


Q4_TILE_ROWS, Q4_TILE_K, Q4_TILE_BYTES = 128, 64, 128 * 32 + 128 * 4


def to_tiled_q4(qw_dev: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Tile records of the tensor-core GEMM: ``qw_dev [..., N, K/8]`` (int32, device nibble order) and
    ``scale [..., N, K/32]`` (fp16, or bf16 for bf16 models: the records keep the two bytes as they are) become ``uint8 [R/128, K/64, 4608]`` where ``R`` is the number of
    rows of all leading slabs stacked (padded to a multiple of 128 with zero scales).  One record holds
    one 128-row x 64-k block: ``[2 halves][128 rows][16 bytes of nibbles]`` followed by
    ``[128 rows][2 fp16 scales]``, so that the kernel streams a whole K sweep of a row block as one
    contiguous range and its threads read shared memory without bank conflicts."""
    k8 = qw_dev.shape[-1]
    if k8 % 8 != 0 or scale.shape[-1] * 4 != k8:
        raise ValueError("tiled int4 layout needs K to be a multiple of 64 and one scale per 32 weights")
    qw2 = qw_dev.reshape(-1, k8)
    if scale.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("tile records hold 16-bit scales")
    sc2 = scale.reshape(-1, scale.shape[-1])
    rows = qw2.shape[0]
    pad = (-rows) % Q4_TILE_ROWS
    if pad:
        qw2 = torch.nn.functional.pad(qw2, (0, 0, 0, pad))
        sc2 = torch.nn.functional.pad(sc2, (0, 0, 0, pad))
    nb, kb = qw2.shape[0] // Q4_TILE_ROWS, k8 // 8
    nib = qw2.reshape(nb, Q4_TILE_ROWS, kb, 2, 4).permute(0, 2, 3, 1, 4).contiguous()
    nib = nib.view(torch.uint8).reshape(nb, kb, Q4_TILE_ROWS * 32)
    scl = sc2.reshape(nb, Q4_TILE_ROWS, kb, 2).permute(0, 2, 1, 3).contiguous()
    scl = scl.view(torch.uint8).reshape(nb, kb, Q4_TILE_ROWS * 4)
    return torch.cat([nib, scl], dim=-1).contiguous()


# ----------------------------------------------------------------------------- fp8
FP8_MAX = {"float8_e4m3fn": 448.0, "float8_e5m2": 57344.0}
_FP8_DT = {"float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2}


def fp8_block_quantize(w: torch.Tensor, block: Tuple[int, int] = (128, 128),
                       dtype: str = "float8_e4m3fn") -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [N, K]`` -> (fp8 weight, ``weight_scale_inv`` fp32 [ceil(N/bn), ceil(K/bk)]) with
    ``w ~= fp8 * scale_inv`` per block (DeepSeek-V3 checkpoint convention)."""
    n, k = w.shape[-2:]
    bn, bk = block
    pn, pk = (-n) % bn, (-k) % bk
    wp = torch.nn.functional.pad(w.float(), (0, pk, 0, pn))
    nb, kb = wp.shape[-2] // bn, wp.shape[-1] // bk
    blocks = wp.reshape(*w.shape[:-2], nb, bn, kb, bk)
    amax = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-12)
    scale_inv = amax / FP8_MAX[dtype]
    qb = blocks / scale_inv.unsqueeze(-1).unsqueeze(-3)
    qw = qb.reshape(*w.shape[:-2], nb * bn, kb * bk)[..., :n, :k].to(_FP8_DT[dtype])
    return qw, scale_inv.to(torch.float32)


def fp8_block_dequantize(qw: torch.Tensor, scale_inv: torch.Tensor,
                         block: Tuple[int, int] = (128, 128),
                         out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    n, k = qw.shape[-2:]
    bn, bk = block
    s = scale_inv.repeat_interleave(bn, dim=-2).repeat_interleave(bk, dim=-1)[..., :n, :k]
    return (qw.to(torch.float32) * s).to(out_dtype)


def fp8_rowwise_group_quantize(x: torch.Tensor, group: int = 128,
                               dtype: str = "float8_e4m3fn") -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row, per-``group`` activation quantisation: scale = amax / fp8_max
    (``block_scale_quantization.py:603-700``). Returns (fp8 x, scale fp32 [..., K/group])."""
    *lead, k = x.shape
    pk = (-k) % group
    xp = torch.nn.functional.pad(x.float(), (0, pk))
    xg = xp.reshape(*lead, -1, group)
    scale = (xg.abs().amax(dim=-1) / FP8_MAX[dtype]).clamp_min(1e-10)
    q = (xg / scale.unsqueeze(-1)).reshape(*lead, -1)[..., :k].to(_FP8_DT[dtype])
    return q, scale


def fp8_per_tensor_quantize(w: torch.Tensor, dtype: str = "float8_e4m3fn"
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q_weight`` fp8 plus scalar fp32 ``q_scale`` with ``w ~= q_weight * q_scale``."""
    amax = w.abs().max().float().clamp_min(1e-12)
    scale = amax / FP8_MAX[dtype]
    return (w.float() / scale).to(_FP8_DT[dtype]), scale.reshape(1)
