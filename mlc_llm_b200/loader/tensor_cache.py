"""Reader / writer of the converted-weight format: ``tensor-cache.json`` + ``params_shard_*.bin``.

Layout (the tvmjs tensor cache the reference writes through ``tvmjs.dump_tensor_cache`` in
``interface/convert_weight.py:190-196``; consumers: ``cpp/multi_gpu/multi_gpu_loader.cc:152-314``,
``support/download_cache.py:183-192``)::

    {"metadata": {"ParamSize": n, "ParamBytes": b, "BitsPerParam": x, ...},
     "records": [{"dataPath": "params_shard_0.bin", "format": "raw-shard", "nbytes": N,
                  "md5sum": "...", "records": [
                      {"name": "...", "shape": [..], "dtype": "float16", "format": "raw" |
                       "f32-to-bf16", "nbytes": n, "byteOffset": o}, ...]}, ...]}

Tensors are packed back to back; ``f32-to-bf16`` stores the upper 16 bits of float32 values and is
widened again on load.  Pre-sharded checkpoints name tensors ``{param}_shard-{rank}``
(``support/preshard.py:16-17``).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import torch

SHARD_BYTES = 32 * 1024 * 1024

_NP = {
    "float32": np.float32, "float16": np.float16, "int32": np.int32, "uint32": np.uint32,
    "int8": np.int8, "uint8": np.uint8, "int64": np.int64, "uint16": np.uint16, "int16": np.int16,
    "bfloat16": np.uint16, "float8_e4m3fn": np.uint8, "float8_e5m2": np.uint8, "bool": np.bool_,
}
_TORCH = {
    "float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
    "int32": torch.int32, "uint32": torch.int32, "int8": torch.int8, "uint8": torch.uint8,
    "int64": torch.int64, "float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2,
    "int16": torch.int16, "uint16": torch.int16, "bool": torch.bool,
}
_NAME = {v: k for k, v in _TORCH.items() if k not in ("uint32", "uint16")}


def dtype_name(t: torch.Tensor, logical: Optional[str] = None) -> str:
    return logical or _NAME[t.dtype]


def _to_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16,):
        return t.view(torch.int16).numpy().tobytes()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy().tobytes()
    return t.numpy().tobytes()


def _from_bytes(buf: memoryview, dtype: str, shape: List[int], fmt: str) -> torch.Tensor:
    if fmt == "f32-to-bf16":
        half = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
        return torch.from_numpy(half.view(np.float32).reshape(shape).copy())
    arr = np.frombuffer(buf, dtype=_NP[dtype]).reshape(shape).copy()
    if dtype == "bfloat16":
        return torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
    if dtype in ("float8_e4m3fn", "float8_e5m2"):
        return torch.from_numpy(arr).view(_TORCH[dtype])
    if dtype == "uint32":
        return torch.from_numpy(arr.view(np.int32))
    if dtype == "uint16":
        return torch.from_numpy(arr.view(np.int16))
    return torch.from_numpy(arr)


def dump_tensor_cache(params: Iterator[Tuple[str, torch.Tensor]], out_dir: str,
                      metadata: Optional[Dict] = None, encode_format: str = "f32-to-bf16",
                      logical_dtypes: Optional[Dict[str, str]] = None,
                      shard_bytes: int = SHARD_BYTES) -> Dict:
    """Write ``(name, tensor)`` pairs as a tensor cache under ``out_dir``; returns the JSON dict.
    ``logical_dtypes`` can relabel a tensor (e.g. int32 storage declared as ``uint32``)."""
    os.makedirs(out_dir, exist_ok=True)
    logical_dtypes = logical_dtypes or {}
    shards: List[Dict] = []
    cur: List[Dict] = []
    buf = bytearray()
    total_params = 0
    total_bytes = 0

    def flush():
        nonlocal cur, buf
        if not cur:
            return
        name = f"params_shard_{len(shards)}.bin"
        with open(os.path.join(out_dir, name), "wb") as f:
            f.write(buf)
        shards.append({"dataPath": name, "format": "raw-shard", "nbytes": len(buf),
                       "records": cur, "md5sum": hashlib.md5(buf).hexdigest()})
        cur, buf = [], bytearray()

    for name, t in params:
        fmt = "raw"
        dt = dtype_name(t, logical_dtypes.get(name))
        if t.dtype == torch.float32 and encode_format == "f32-to-bf16":
            raw = _f32_to_bf16_bytes(t)
            fmt = "f32-to-bf16"
        else:
            raw = _to_bytes(t)
        if buf and len(buf) + len(raw) > shard_bytes:
            flush()
        cur.append({"name": name, "shape": list(t.shape), "dtype": dt, "format": fmt,
                    "nbytes": len(raw), "byteOffset": len(buf)})
        buf += raw
        total_params += t.numel()
        total_bytes += len(raw)
    flush()
    meta = dict(metadata or {})
    meta.setdefault("ParamSize", total_params)
    meta.setdefault("ParamBytes", float(total_bytes))
    doc = {"metadata": meta, "records": shards}
    with open(os.path.join(out_dir, "tensor-cache.json"), "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=2)
    return doc


def _f32_to_bf16_bytes(t: torch.Tensor) -> bytes:
    """fp32 -> bf16 bit patterns with round-to-nearest-even, as the tvmjs writer of the reference's
    artifacts does for finite values; Inf / NaN keep their upper half (adding the rounding bias to
    them could carry into the sign / exponent)."""
    u = t.detach().cpu().contiguous().numpy().view(np.uint32)
    finite = (u & np.uint32(0x7F800000)) != np.uint32(0x7F800000)
    bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    rounded = (u.astype(np.uint64) + bias.astype(np.uint64)) >> np.uint64(16)
    out = np.where(finite, rounded, (u >> np.uint32(16)).astype(np.uint64))
    return out.astype(np.uint16).tobytes()


def update_tensor_cache(params: Iterator[Tuple[str, torch.Tensor]], out_dir: str,
                        encode_format: str = "f32-to-bf16") -> Dict:
    """Add (or replace) tensors in the tensor cache under ``out_dir`` without rewriting its existing
    shards: the new tensors go to one extra shard file and records of the same name in older shards are
    dropped from the index.  Creates the cache when there is none."""
    index = os.path.join(out_dir, "tensor-cache.json")
    if not os.path.isfile(index):
        return dump_tensor_cache(params, out_dir, encode_format=encode_format)
    with open(index, encoding="utf-8") as f:
        doc = json.load(f)
    items = list(params)
    names = {n for n, _ in items}
    buf = bytearray()
    records: List[Dict] = []
    for name, t in items:
        fmt = "raw"
        if t.dtype == torch.float32 and encode_format == "f32-to-bf16":
            raw = _f32_to_bf16_bytes(t)
            fmt = "f32-to-bf16"
        else:
            raw = _to_bytes(t)
        records.append({"name": name, "shape": list(t.shape), "dtype": dtype_name(t), "format": fmt,
                        "nbytes": len(raw), "byteOffset": len(buf)})
        buf += raw
    for shard in doc["records"]:
        shard["records"] = [r for r in shard["records"] if r["name"] not in names]
    used = {s["dataPath"] for s in doc["records"]}
    k = 0
    while f"params_shard_extra_{k}.bin" in used:
        k += 1
    path = f"params_shard_extra_{k}.bin"
    with open(os.path.join(out_dir, path), "wb") as f:
        f.write(buf)
    doc["records"].append({"dataPath": path, "format": "raw-shard", "nbytes": len(buf), "records": records,
                           "md5sum": hashlib.md5(buf).hexdigest()})
    # the totals describe the records the index still names, not what the shard files hold
    live = [r for shard in doc["records"] for r in shard["records"]]
    meta = doc.setdefault("metadata", {})
    meta["ParamSize"] = int(sum(int(np.prod(r["shape"], dtype=np.int64)) for r in live))
    meta["ParamBytes"] = float(sum(r["nbytes"] for r in live))
    with open(index, "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=2)
    return doc


class TensorCache:
    """Lazy reader: iterates shard by shard so peak host memory is one shard file."""

    def __init__(self, model_dir: str, verify_md5: bool = False):
        self.dir = model_dir
        path = os.path.join(model_dir, "tensor-cache.json")
        if not os.path.exists(path):
            legacy = os.path.join(model_dir, "ndarray-cache.json")
            path = legacy if os.path.exists(legacy) else path
        with open(path, encoding="utf-8") as f:
            self.doc = json.load(f)
        self.verify_md5 = verify_md5
        self.index: Dict[str, Tuple[int, int]] = {}
        for si, shard in enumerate(self.doc["records"]):
            for ri, rec in enumerate(shard["records"]):
                self.index[rec["name"]] = (si, ri)

    @property
    def metadata(self) -> Dict:
        return self.doc.get("metadata", {})

    def names(self) -> List[str]:
        return list(self.index)

    def _read_shard(self, si: int) -> bytes:
        shard = self.doc["records"][si]
        with open(os.path.join(self.dir, shard["dataPath"]), "rb") as f:
            data = f.read()
        if self.verify_md5 and "md5sum" in shard and hashlib.md5(data).hexdigest() != shard["md5sum"]:
            raise ValueError(f"md5 mismatch for {shard['dataPath']}")
        return data

    def __iter__(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for si, shard in enumerate(self.doc["records"]):
            view = memoryview(self._read_shard(si))
            for rec in shard["records"]:
                off, n = rec["byteOffset"], rec["nbytes"]
                yield rec["name"], _from_bytes(view[off:off + n], rec["dtype"], rec["shape"],
                                               rec.get("format", "raw"))

    def get(self, name: str) -> torch.Tensor:
        si, ri = self.index[name]
        rec = self.doc["records"][si]["records"][ri]
        view = memoryview(self._read_shard(si))
        off, n = rec["byteOffset"], rec["nbytes"]
        return _from_bytes(view[off:off + n], rec["dtype"], rec["shape"], rec.get("format", "raw"))
