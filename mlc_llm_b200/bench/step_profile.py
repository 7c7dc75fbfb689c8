"""Per-operator time breakdown of one prefill step and one decode step of a model.

``python -m mlc_llm_b200.bench.step_profile --model llama-3-8b --quant q4f16_1 --batch 256 --ctx 640``

Every call of an ``ops`` function is bracketed by CUDA events (with a synchronise, so this measures
kernels back to back without overlap) and summed per operator and call-site shape.  The output shows
which kernel a serving step spends its time in and what launch overhead the Python driver adds
(wall time of the step minus the sum of kernel times).
"""

from __future__ import annotations

import argparse
import collections
import json
import time

import numpy as np
import torch

from .. import _core, ops
from .. import quantization as Q
from ..models import config as mc
from ..models import loader
from ..models.presets import MODEL_PRESETS
from ..models.transformer import DecoderModel
from ..serve.executor import ModelExecutor

_TIMED = ["linear", "rmsnorm", "add_rmsnorm", "act_mul", "embed", "rope_append", "paged_attention",
          "argmax", "row_gather"]


class OpTimer:
    def __init__(self):
        self.totals = collections.defaultdict(float)
        self.counts = collections.defaultdict(int)
        self.enabled = False
        self._orig = {}

    def install(self):
        import mlc_llm_b200.models.transformer as tr  # pylint: disable=import-outside-toplevel

        for name in _TIMED:
            fn = getattr(ops, name)
            self._orig[name] = fn

            def wrapped(*args, _fn=fn, _name=name, **kwargs):
                if not self.enabled:
                    return _fn(*args, **kwargs)
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                out = _fn(*args, **kwargs)
                e.record()
                torch.cuda.synchronize()
                key = _name
                if _name == "linear":
                    lw = args[1]
                    key = f"linear[{args[0].shape[0]}x{lw.out_features}x{lw.in_features},{lw.kind}]"
                self.totals[key] += s.elapsed_time(e)
                self.counts[key] += 1
                return out

            setattr(ops, name, wrapped)
        _ = tr


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--quant", default="q4f16_1")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=640)
    ap.add_argument("--prefill-tokens", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = preset)")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    hf = dict(MODEL_PRESETS[args.model])
    if args.layers:
        hf["num_hidden_layers"] = args.layers
    cfg = mc.from_dict(hf["model_type"], hf)
    quant = Q.get(args.quant)
    store = loader.random_params(cfg, quant, 0, dev)
    model = DecoderModel(cfg, quant, store, dev)
    pages = (args.batch * (args.ctx + 32) + args.prefill_tokens) // 16 + 2 * args.batch + 64
    model.create_kv_cache(pages, 16)
    ex = ModelExecutor([model], dev)
    kv = _core.KVManager(pages, 16, args.batch + 64)
    timer = OpTimer()
    timer.install()
    rng = np.random.default_rng(0)
    greedy = {"logit_token_index": None, "temperature": None, "top_p": None, "top_k": None, "uniform": None,
              "penalties": None, "pen_row": [], "pen_token": [], "pen_count": [], "bias_row": [],
              "bias_token": [], "bias_value": [], "mask_rows": [], "mask_bits": [], "num_top_logprobs": 0,
              "prob_slots": []}

    def sp_for(rows):
        n = len(rows)
        d = dict(greedy)
        d.update(logit_token_index=np.asarray(rows, dtype=np.int32), temperature=np.zeros(n, np.float32),
                 top_p=np.ones(n, np.float32), top_k=np.zeros(n, np.int32), uniform=np.zeros(n, np.float32),
                 penalties=np.tile(np.asarray([0, 0, 1], np.float32), n))
        return d

    # fill the cache: sequences of ctx tokens, prefilled in chunks
    ids = list(range(args.batch))
    for i in ids:
        kv.add_sequence(i)
    per = max(1, args.prefill_tokens // args.ctx)
    report = {}
    for start in range(0, args.batch, per):
        group = ids[start:start + per]
        lens = [args.ctx] * len(group)
        plan = kv.begin_forward(group, lens)
        toks = rng.integers(0, 32000, sum(lens)).astype(np.int32)
        rows = np.cumsum(lens) - 1
        last = start + per >= args.batch
        if last:
            torch.cuda.synchronize()
            timer.enabled = True
            t0 = time.perf_counter()
        ex.forward_sample(0, plan, toks, None, sp_for(rows))
        if last:
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) * 1e3
            timer.enabled = False
            report["prefill"] = {"tokens": int(sum(lens)), "wall_ms_with_sync_per_op": wall,
                                 "ops": {k: round(v, 3) for k, v in sorted(timer.totals.items(), key=lambda x: -x[1])}}
            timer.totals.clear()
            timer.counts.clear()
    # decode steps
    def decode_step():
        plan = kv.begin_forward(ids, [1] * args.batch)
        toks = rng.integers(0, 32000, args.batch).astype(np.int32)
        return ex.forward_sample(0, plan, toks, None, sp_for(list(range(args.batch))))

    for _ in range(3):
        decode_step()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    s.record()
    for _ in range(5):
        decode_step()
    e.record()
    torch.cuda.synchronize()
    report["decode_untimed_ops"] = {"device_ms_per_step": s.elapsed_time(e) / 5,
                                    "wall_ms_per_step": (time.perf_counter() - t0) * 1e3 / 5}
    graphs, ex.use_graphs = ex.use_graphs, False  # a graph replay would hide the operators from the timer
    timer.enabled = True
    decode_step()
    timer.enabled = False
    ex.use_graphs = graphs
    report["decode"] = {"batch": args.batch, "ctx": args.ctx,
                        "kernel_ms_sum": round(sum(timer.totals.values()), 3),
                        "ops": {k: [round(v, 3), timer.counts[k]] for k, v in
                                sorted(timer.totals.items(), key=lambda x: -x[1])}}
    print(json.dumps(report, indent=1))
    if args.out:
        with open(args.out, "w", encoding="utf-8") as f:
            json.dump(report, f, indent=1)
    ops.check_status(dev)


if __name__ == "__main__":
    main()
