"""``python -m mlc_llm_b200.testing.debug_compare``: run a prompt on one device and re-run every
operator call on a second device with the same inputs, reporting where the two disagree (reference:
``python/mlc_llm/testing/debug_compare.py``, ``LibCompare``: each kernel of one library is re-run
through another library / device and compared).

The typical use is CUDA kernels against the CPU reference operators:

    python -m mlc_llm_b200.testing.debug_compare "hello" --model random://tiny-llama-gpu?quant=q4f16_1 \\
        --device cuda --cmp-device cpu
"""

from __future__ import annotations

import argparse
import copy
import os
from typing import Any, Dict, List

import torch

from .instrument import tap_ops


def _move(v: Any, device: torch.device) -> Any:
    if isinstance(v, torch.Tensor):
        t = v.detach().to(device)
        return t.clone() if t.device == v.device else t
    if hasattr(v, "to") and hasattr(v, "kind") and hasattr(v, "w"):  # LinearWeight (re-laid out per device)
        return v.to(device)
    if isinstance(v, (list, tuple)):
        return type(v)(_move(x, device) for x in v)
    if hasattr(v, "__dict__") and not callable(v):  # plans / small records of tensors
        c = copy.copy(v)
        for k, x in vars(v).items():
            setattr(c, k, _move(x, device))
        return c
    return v


class OpCompare:
    """``before`` copies the inputs to the comparison device (operators may update their inputs in
    place); ``after`` runs the same operator there and records the largest deviation."""

    def __init__(self, cmp_device: str, rtol: float = 1e-2, atol: float = 1e-2):
        self.cmp_device = torch.device(cmp_device)
        self.rtol, self.atol = rtol, atol
        self.records: List[Dict[str, Any]] = []
        self._originals: Dict[str, Any] = {}
        self._busy = False

    def before(self, name, args, kwargs):
        if self._busy:
            return None
        return (_move(list(args), self.cmp_device), {k: _move(v, self.cmp_device) for k, v in kwargs.items()})

    def after(self, name, args, kwargs, result, token) -> None:
        if token is None or self._busy:
            return
        from .. import ops  # pylint: disable=import-outside-toplevel

        self._busy = True  # operators call each other: compare the outermost call only
        try:
            fn = self._originals.get(name) or getattr(ops, name)
            want = fn(*token[0], **token[1])
        finally:
            self._busy = False
        got_t = [t for t in (result if isinstance(result, (list, tuple)) else [result]) if isinstance(t, torch.Tensor)]
        want_t = [t for t in (want if isinstance(want, (list, tuple)) else [want]) if isinstance(t, torch.Tensor)]
        worst, ok = 0.0, True
        for g, w in zip(got_t, want_t):
            g32, w32 = g.detach().float().cpu(), w.detach().float().cpu()
            if g32.shape != w32.shape:
                ok = False
                continue
            if g32.numel():
                worst = max(worst, float((g32 - w32).abs().max()))
                ok = ok and bool(torch.allclose(g32, w32, rtol=self.rtol, atol=self.atol))
        self.records.append({"op": name, "index": len(self.records), "max_abs_err": worst, "ok": ok})

    def summary(self) -> Dict[str, Dict[str, Any]]:
        out: Dict[str, Dict[str, Any]] = {}
        for r in self.records:
            s = out.setdefault(r["op"], {"calls": 0, "max_abs_err": 0.0, "mismatches": 0})
            s["calls"] += 1
            s["max_abs_err"] = max(s["max_abs_err"], r["max_abs_err"])
            s["mismatches"] += 0 if r["ok"] else 1
        return out


def compare(model: str, prompt, device: str, cmp_device: str, generate_len: int = 2,
            rtol: float = 1e-2, atol: float = 1e-2) -> OpCompare:
    from ..serve.config import EngineConfig  # pylint: disable=import-outside-toplevel
    from ..serve.sync_engine import SyncMLCEngine  # pylint: disable=import-outside-toplevel

    saved = {k: os.environ.get(k) for k in ("MLCB_CUDA_GRAPH", "MLCB_PIPELINED_DECODE")}
    os.environ["MLCB_CUDA_GRAPH"] = "0"  # graph replays would bypass the operator layer
    os.environ["MLCB_PIPELINED_DECODE"] = "0"  # one engine step = one model call = one token
    try:
        eng = SyncMLCEngine(model, device, engine_config=EngineConfig(mode="local", max_num_sequence=1,
                                                                       prefix_cache_mode="disable"))
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    cmp = OpCompare(cmp_device, rtol, atol)
    from .. import ops  # pylint: disable=import-outside-toplevel
    from .instrument import DEFAULT_OPS  # pylint: disable=import-outside-toplevel

    # attention and KV append read the paged pool: comparing them would copy the pool per call
    names = [n for n in DEFAULT_OPS if n not in ("rope_append", "paged_attention")]
    cmp._originals = {n: getattr(ops, n) for n in names if hasattr(ops, n)}  # pylint: disable=protected-access
    toks = eng.tokenizer.encode(prompt) if isinstance(prompt, str) else list(prompt)
    with tap_ops(before=cmp.before, after=cmp.after, names=names):
        eng.generate([toks], {"max_tokens": generate_len, "temperature": 0.0, "debug_config": {"ignore_eos": True}})
    return cmp


def main(argv=None) -> None:
    p = argparse.ArgumentParser("mlc_llm_b200.testing.debug_compare")
    p.add_argument("prompt", type=str)
    p.add_argument("--model", type=str, required=True)
    p.add_argument("--device", type=str, default="auto")
    p.add_argument("--cmp-device", type=str, default="cpu")
    p.add_argument("--generate-len", type=int, default=2)
    p.add_argument("--rtol", type=float, default=1e-2)
    p.add_argument("--atol", type=float, default=1e-2)
    a = p.parse_args(argv)
    cmp = compare(a.model, a.prompt, a.device, a.cmp_device, a.generate_len, a.rtol, a.atol)
    for op, s in sorted(cmp.summary().items()):
        flag = "" if not s["mismatches"] else f"   <-- {s['mismatches']} mismatching calls"
        print(f"{op:22s} calls {s['calls']:4d}   max |err| {s['max_abs_err']:.3e}{flag}")


if __name__ == "__main__":
    main()
