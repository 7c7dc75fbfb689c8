"""Headline serving benchmark: output tokens/s of continuous-batching generation.

Workload (one "step" = one full pass of it): Llama-3-8B, q4f16_1 weights (random init, N(0, 0.02),
seeded), 256 requests of 512 uniform-random prompt tokens, 256 output tokens each (EOS ignored),
16-token KV pages, fp16 KV cache, greedy sampling.  With N > 1 GPUs the model runs tensor-parallel
over the N ranks (one process per GPU, NCCL); the request count is fixed, so scaling is "strong".

Two numbers are reported:
* ``value``  -- device-timed (CUDA events on the compute stream, max over ranks) run of the native
  engine stepped directly through the step-driven ``SyncMLCEngine``;
* ``e2e``    -- the same workload through the public ``MLCEngine.completions`` API (background engine
  thread, stream-back thread, detokenisation), wall-clock, including per-step H2D of the step's
  index arrays from pinned memory and D2H of the sampled tokens.

``--config`` selects one of the target workloads (the default, 2, is the headline):

* ``2``      Llama-3-8B q4f16_1, tensor parallel over the N ranks, 256 x 512 -> 256;
* ``3``      Llama-3-70B bf16, tensor parallel over N ranks (meant for 8), 512 requests with prompt lengths
             uniform in [128, 2048] and 512 output tokens;
* ``3-fp8``  the same with block-scaled e4m3 weights;
* ``4``      Mixtral-8x7B bf16 with the experts sharded over the ranks (all-to-all dispatch / combine),
             256 x 1024 -> 256;
* ``5``      Llama-3-70B bf16 on 2 pipeline stages x N/2 tensor-parallel ranks with the prefix cache on
             (64 requests share a 1536-token prefix, 128-token suffixes) and speculative decoding (a random
             2-layer draft model proposing 4 tokens per step), 256 output tokens.

``--impl reference`` would run the unmodified reference implementation; it cannot be installed in
this environment (its build needs the TVM / tokenizers-cpp / xgrammar submodules, which are empty
directories), so that arm prints an ``unavailable`` line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np


def _reference_arm():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "offline pip install of the reference fails at CMake: 3rdparty/tvm, "
                       "3rdparty/tokenizers-cpp and 3rdparty/xgrammar are empty submodule directories "
                       "(add_subdirectory has no CMakeLists.txt); apache-tvm-ffi is not in the wheelhouse",
    }))
    return 0


# The target workloads. prompt_len is (low, high): lengths are uniform in that range.
WORKLOADS = {
    "2": dict(model="llama-3-8b", quant="q4f16_1", requests=256, prompt_len=(512, 512), output_len=256,
              tp1_check=True),
    "3": dict(model="llama-3-70b", quant="q0bf16", requests=512, prompt_len=(128, 2048), output_len=512),
    "3-fp8": dict(model="llama-3-70b", quant="fp8_e4m3fn_bf16_block_scale", requests=512, prompt_len=(128, 2048),
                  output_len=512),
    "4": dict(model="mixtral-8x7b", quant="q0bf16", requests=256, prompt_len=(1024, 1024), output_len=256,
              model_args="&expert_parallel=true"),
    "5": dict(model="llama-3-70b", quant="q0bf16", requests=64, prompt_len=(128, 128), output_len=256,
              shared_prefix=1536, pipeline_stages=2, draft="llama-3-draft-2l", draft_length=4),
}


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    cols = [c.strip() for c in line.split(",")]
                    if len(cols) < 9:
                        continue
                    try:
                        sm.append(float(cols[1]))
                        mx.append(float(cols[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                          "sw_power_cap"), cols[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", default="2", choices=sorted(WORKLOADS))
    ap.add_argument("--model", default=None)
    ap.add_argument("--quant", default=None)
    ap.add_argument("--requests", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--output-len", type=int, default=None)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--tp1-check", choices=("auto", "on", "off"), default="auto",
                    help="at N > 1: compare 8 fixed greedy requests with a 1-rank run of the same weights "
                         "(auto: only for models whose unsharded copy is cheap to build)")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return _reference_arm()
    wl = dict(WORKLOADS[args.config])
    for k in ("model", "quant", "requests", "output_len"):
        if getattr(args, k) is not None:
            wl[k] = getattr(args, k)
    if args.prompt_len is not None:
        wl["prompt_len"] = (args.prompt_len, args.prompt_len)
    args.model, args.quant, args.requests, args.output_len = wl["model"], wl["quant"], wl["requests"], wl["output_len"]
    lo, hi = wl["prompt_len"]
    args.prompt_len = hi

    import torch

    from mlc_llm_b200 import parallel
    from mlc_llm_b200.ops import _lib
    from mlc_llm_b200.serve.config import EngineConfig

    rank, world, local = parallel.env_world()
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            raise SystemExit("for --gpus N > 1 launch with torch.distributed.run --nproc-per-node N")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    pp = int(wl.get("pipeline_stages", 1)) if world > 1 else 1
    if world % pp:
        raise SystemExit(f"config {args.config} needs a multiple of {pp} GPUs")
    comm = parallel.Communicator(tp_size=world // pp, pp_size=pp) if world > 1 else None
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)

    model = f"random://{args.model}?quant={args.quant}&seed=0{wl.get('model_args', '')}"
    shared = int(wl.get("shared_prefix", 0))
    total_tokens = args.requests * (shared + args.prompt_len + args.output_len)
    extra = {}
    if wl.get("draft"):
        extra = dict(additional_models=[f"random://{wl['draft']}?quant={args.quant}&seed=1"],
                     speculative_mode="small_draft", spec_draft_length=int(wl["draft_length"]))
    cfg = EngineConfig(mode="server", max_num_sequence=args.requests, prefill_chunk_size=8192,
                       max_total_sequence_length=total_tokens + 16 * args.requests + 8192,
                       prefix_cache_mode="radix" if shared else "disable", gpu_memory_utilization=0.90,
                       tensor_parallel_shards=world // pp if world > 1 else None,
                       pipeline_parallel_stages=pp if pp > 1 else None, **extra)
    rng = np.random.default_rng(1234)
    gen_cfg = {"max_tokens": args.output_len, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    vocab_hi = 32000

    # correctness line at N > 1 (outside the timed region): 8 fixed greedy requests, 32 tokens each, through
    # the N-rank engine and, after the ranks have parted, through a 1-rank engine of the same weights
    tp1_check = world > 1 and pp == 1 and (args.tp1_check == "on" or
                                           (args.tp1_check == "auto" and wl.get("tp1_check", False)))
    check_rng = np.random.default_rng(99)
    check_prompts = [check_rng.integers(0, vocab_hi, 64).tolist() for _ in range(8)]
    check_cfg = {"max_tokens": 32, "temperature": 0.0, "debug_config": {"ignore_eos": True}}

    def make_prompts():
        # fresh prompts every pass so no pass benefits from an earlier one (a shared prefix is shared
        # within a pass only)
        prefix = rng.integers(0, vocab_hi, shared).tolist() if shared else []
        lens = rng.integers(lo, hi + 1, args.requests)
        return [prefix + rng.integers(0, vocab_hi, int(n)).tolist() for n in lens]

    # ------------------------------------------------------------------ worker ranks
    if rank != 0:
        from mlc_llm_b200.serve.engine_base import EngineRuntime

        cfg.model = model
        rt = EngineRuntime(cfg, device, comm=comm)
        passes = (args.warmup + args.steps) * (1 if args.no_e2e else 2) + (1 if tp1_check else 0)
        for _ in range(passes):
            comm.barrier()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            parallel.worker_loop(rt.executor, comm)
            end.record()
            torch.cuda.synchronize()
            comm.barrier()
            comm.max_over_ranks(start.elapsed_time(end))
        comm.destroy()
        return 0

    # ------------------------------------------------------------------ rank 0
    from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

    eng = SyncMLCEngine(model, device, engine_config=cfg, comm=comm)
    lib = _lib.lib()
    lib.mlcb_launch_count.restype = __import__("ctypes").c_longlong

    def run_pass_device():
        prompts = make_prompts()
        if comm is not None:
            comm.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = lib.mlcb_launch_count() + eng.runtime.executor.graph_launches
        start.record()
        out_tokens = eng.run_token_workload(prompts, gen_cfg)
        end.record()
        torch.cuda.synchronize()
        if comm is not None:
            comm.shutdown_workers()
            comm.barrier()
        ms = start.elapsed_time(end)
        if comm is not None:
            ms = comm.max_over_ranks(ms)
        _lib.check_status(device)
        return ms, out_tokens, lib.mlcb_launch_count() + eng.runtime.executor.graph_launches - l0

    for _ in range(args.warmup):
        run_pass_device()
    host0 = dict(eng.runtime.executor.host_times)
    wall0 = time.perf_counter()
    sampler = ClockSampler(local)
    sampler.start()
    times, toks, launches = [], 0, 0
    for _ in range(args.steps):
        ms, n, l = run_pass_device()
        times.append(ms)
        toks += n
        launches += l
    clocks = sampler.stop()
    # where rank 0's host time went per engine step (ms): executor phases, and the rest of the loop
    # (native engine step, plan building, output handling) as "engine_other"
    host1 = eng.runtime.executor.host_times
    calls = max(1.0, host1["calls"] - host0["calls"])
    host_ms = {k: round((host1[k] - host0[k]) * 1e3 / calls, 3) for k in host1 if k != "calls"}
    host_ms["engine_other"] = round((time.perf_counter() - wall0) * 1e3 / calls - sum(host_ms.values()), 3)
    total_ms = sum(times)
    value = toks / (total_ms / 1e3)
    steps_per_pass = json.loads(eng.debug_stats())
    engine_steps = steps_per_pass["num_prefill_steps"] + steps_per_pass["num_decode_steps"]
    # the native engine's own split of a decode step's host time (ms per decode step, all passes so far)
    native_ms = {k: round(v * 1e3 / max(1, steps_per_pass["num_decode_steps"]), 3)
                 for k, v in steps_per_pass.get("decode_host_seconds", {}).items()}

    check_tokens = None
    if tp1_check:
        comm.barrier()
        _, check_out = eng.generate(check_prompts, check_cfg)
        check_tokens = [t[0] for t in check_out]
        torch.cuda.synchronize()
        comm.shutdown_workers()
        comm.barrier()
        comm.max_over_ranks(0.0)

    # ------------------------------------------------------------------ end to end, public API
    e2e = None
    if not args.no_e2e:
        h2d0, d2h0 = eng.runtime.executor.h2d_bytes, eng.runtime.executor.d2h_bytes
        steps0 = json.loads(eng.debug_stats())
        from mlc_llm_b200.serve.engine import MLCEngine

        api = MLCEngine.from_runtime(eng.runtime)

        lat = []  # per-request server-side latencies (engine metrics: ttft_s, decode_tokens_per_s)

        def run_pass_api():
            prompts = make_prompts()
            if comm is not None:
                comm.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = api.generate_many(prompts, gen_cfg)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if comm is not None:
                comm.shutdown_workers()
                comm.barrier()
                comm.max_over_ranks(0.0)
            lat.extend((r["usage"].get("extra") or {}) for r in res)
            return dt, sum(r["usage"]["completion_tokens"] for r in res)

        for _ in range(args.warmup):
            run_pass_api()
        h2d0, d2h0 = eng.runtime.executor.h2d_bytes, eng.runtime.executor.d2h_bytes
        st0 = api.debug_step_count()
        dts, etoks = [], 0
        lat.clear()
        for _ in range(args.steps):
            dt, n = run_pass_api()
            dts.append(dt)
            etoks += n
        nsteps = max(1, api.debug_step_count() - st0)
        e2e = {"value": etoks / sum(dts), "unit": "output tokens/s",
               "h2d_bytes_per_step": (eng.runtime.executor.h2d_bytes - h2d0) / nsteps,
               "d2h_bytes_per_step": (eng.runtime.executor.d2h_bytes - d2h0) / nsteps,
               "engine_steps": nsteps}
        ttft = sorted(x["ttft_s"] for x in lat if "ttft_s" in x)
        tpot = sorted(1.0 / x["decode_tokens_per_s"] for x in lat if x.get("decode_tokens_per_s"))
        if ttft:
            e2e["p50_ttft_s"] = ttft[len(ttft) // 2]
        if tpot:
            e2e["p50_tpot_s"] = tpot[len(tpot) // 2]
        api.terminate()

    line = {
        "metric": "output tok/s (device-timed, max over ranks)",
        "value": value, "unit": "output tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp16 activations, int4-group weights (q4f16_1)"
        if args.quant == "q4f16_1" else ("bf16" if args.quant == "q0bf16" else args.quant), "data": "synthetic (uniform-random token ids, random-init weights)",
        "config": {"workload": args.config, "model": f"{args.model} {args.quant}", "global_batch": args.requests,
                   "seq_len": shared + args.prompt_len + args.output_len,
                   "prompt_len": args.prompt_len if lo == hi else f"uniform[{lo},{hi}]", "shared_prefix": shared,
                   "output_len": args.output_len,
                   "parallelism": (f"pp{pp}xtp{world // pp}" if pp > 1 else
                                   (f"ep{world}" if "expert_parallel" in wl.get("model_args", "") and world > 1
                                    else f"tp{world}")),
                   "speculative": f"{wl['draft']} x{wl['draft_length']}" if wl.get("draft") else None,
                   "l2": "inputs larger than L2 (weights and KV cache far exceed 126 MB)",
                   "kv_page": 16, "kv_dtype": "fp16", "sampling": "greedy, ignore_eos"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
        "engine_steps_per_pass": engine_steps // max(1, args.warmup + args.steps),
        "host_ms_per_engine_step": host_ms, "native_engine_ms_per_decode_step": native_ms,
    }
    if comm is not None:
        comm.destroy()
    if check_tokens is not None:
        try:
            import gc

            del eng
            gc.collect()
            torch.cuda.empty_cache()
            os.environ["MLCB_FUSED_TP"] = "0"
            one = SyncMLCEngine(model, device, engine_config=EngineConfig(
                mode="server", max_num_sequence=8, prefill_chunk_size=8192, max_total_sequence_length=4096,
                prefix_cache_mode="disable", gpu_memory_utilization=0.5))
            _, ref_out = one.generate(check_prompts, check_cfg)
            prefix = []
            for a, b in zip(check_tokens, (t[0] for t in ref_out)):
                n = 0
                while n < min(len(a), len(b)) and a[n] == b[n]:
                    n += 1
                prefix.append(n)
            # the ranks add their partial sums in another order than one GPU does, so with random weights a
            # sequence can part ways with the 1-rank run at a near-tie and never return: the first token and the
            # matched prefix length say more than the count of fully equal sequences
            line["tokens_match_tp1"] = {"requests": len(prefix), "tokens_each": 32,
                                        "first_token_equal": sum(1 for n in prefix if n >= 1),
                                        "all_32_equal": sum(1 for n in prefix if n >= 32),
                                        "matched_prefix_lengths": prefix}
        except Exception as err:  # pylint: disable=broad-except
            # the timed result stands on its own: a failed check is reported, not fatal
            line["tokens_match_tp1"] = {"error": str(err)[:200]}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
