"""``python -m mlc_llm_b200.testing.debug_chat``: run one prompt through a model and dump the
arguments and results of every operator call to ``.npz`` files, flagging the first NaN / Inf
(reference: ``python/mlc_llm/testing/debug_chat.py``: ``DefaultDebugInstrument`` and ``DebugChat``).

    python -m mlc_llm_b200.testing.debug_chat "hello" --model random://tiny-llama?quant=q0f32 \\
        --debug-dir /tmp/debug --generate-len 4
"""

from __future__ import annotations

import argparse
import os
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .instrument import tap_ops

MAX_DUMP_BYTES = 1 << 31


class DebugInstrument:
    """Writes ``f<counter>_<op>.npz`` with ``arg_<i>`` / ``out_<i>`` arrays per operator call."""

    def __init__(self, debug_out: str):
        self.reset(debug_out)

    def reset(self, debug_out: str) -> None:
        self.counter = 0
        self.first_nan_occurred = False
        self.first_inf_occurred = False
        self.debug_out = debug_out
        self.log: List[str] = []
        os.makedirs(debug_out, exist_ok=True)

    @staticmethod
    def _tensors(values) -> List[torch.Tensor]:
        out = []
        for v in values:
            if isinstance(v, torch.Tensor):
                out.append(v)
            elif hasattr(v, "w") and isinstance(getattr(v, "w"), torch.Tensor):  # LinearWeight
                out.append(v.w)
            elif isinstance(v, (list, tuple)):
                out.extend(DebugInstrument._tensors(v))
        return out

    @staticmethod
    def _to_numpy(t: torch.Tensor) -> np.ndarray:
        if t.numel() * t.element_size() > MAX_DUMP_BYTES:
            return np.zeros(())  # too large to be worth a file
        t = t.detach()
        if t.dtype in (torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2):
            t = t.float()
        return t.cpu().numpy()

    def __call__(self, name: str, args, kwargs, result, _token=None) -> None:
        if self.first_nan_occurred or self.first_inf_occurred:
            return
        func_name = f"f{self.counter}_{name}"
        arrays: Dict[str, np.ndarray] = {}
        for i, t in enumerate(self._tensors(list(args) + list(kwargs.values()))):
            arrays[f"arg_{i}"] = self._to_numpy(t)
        outs = self._tensors(result if isinstance(result, (list, tuple)) else [result])
        for i, t in enumerate(outs):
            arr = self._to_numpy(t)
            arrays[f"out_{i}"] = arr
            if arr.dtype.kind == "f":
                nans, infs = int(np.isnan(arr).sum()), int(np.isinf(arr).sum())
                if nans:
                    self.log.append(f"{func_name} has NaN: {nans}")
                    self.first_nan_occurred = True
                if infs:
                    self.log.append(f"{func_name} has INF: {infs}")
                    self.first_inf_occurred = True
        np.savez(os.path.join(self.debug_out, func_name + ".npz"), **arrays)
        self.counter += 1


class DebugChat:
    """Single-sequence runner: prefill the prompt, then decode ``generate_len`` tokens greedily, with
    every operator call recorded under ``debug_dir/prefill`` and ``debug_dir/decode_<i>``."""

    def __init__(self, model: str, debug_dir: str, device: str = "auto",
                 instrument: Optional[Any] = None):
        from ..serve.config import EngineConfig  # pylint: disable=import-outside-toplevel
        from ..serve.sync_engine import SyncMLCEngine  # pylint: disable=import-outside-toplevel

        self.debug_dir = debug_dir
        saved = {k: os.environ.get(k) for k in ("MLCB_CUDA_GRAPH", "MLCB_PIPELINED_DECODE")}
        os.environ["MLCB_CUDA_GRAPH"] = "0"  # graph replays would bypass the operator layer
        os.environ["MLCB_PIPELINED_DECODE"] = "0"  # one engine step = one model call = one token
        try:
            self.engine = SyncMLCEngine(model, device, engine_config=EngineConfig(
                mode="local", max_num_sequence=1, prefix_cache_mode="disable"))
        finally:
            for k, v in saved.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
        self.instrument = instrument or DebugInstrument(os.path.join(debug_dir, "prefill"))

    def generate(self, prompt, generate_len: int) -> List[int]:
        """Returns the generated token ids; ``prompt`` is text or a list of token ids."""
        eng = self.engine
        toks = eng.tokenizer.encode(prompt) if isinstance(prompt, str) else list(prompt)
        cfg = {"max_tokens": generate_len, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
        eng.add_request("debug-chat", [toks], cfg)
        out: List[int] = []
        step = 0
        with tap_ops(after=self.instrument):
            while not eng.empty():
                self.instrument.reset(os.path.join(self.debug_dir, "prefill" if step == 0 else f"decode_{step - 1}"))
                eng.step()
                for o in eng.take_outputs():
                    out.extend(o["group_delta_token_ids"][0])
                for line in getattr(self.instrument, "log", []):
                    print(line)
                step += 1
        return out


def main(argv=None) -> None:
    p = argparse.ArgumentParser("mlc_llm_b200.testing.debug_chat")
    p.add_argument("prompt", type=str)
    p.add_argument("--model", type=str, required=True)
    p.add_argument("--device", type=str, default="auto")
    p.add_argument("--debug-dir", type=str, required=True)
    p.add_argument("--generate-len", type=int, default=8)
    a = p.parse_args(argv)
    chat = DebugChat(a.model, a.debug_dir, a.device)
    ids = chat.generate(a.prompt, a.generate_len)
    print("generated token ids:", ids)
    print("text:", chat.engine.tokenizer.decode(ids))


if __name__ == "__main__":
    main()
