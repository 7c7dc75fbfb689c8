"""Kernel timeline of decode steps of the serving engine, from the CUDA activity records of
``torch.profiler`` (CUPTI), on one GPU or tensor-parallel over several.

``python -m mlc_llm_b200.bench.decode_timeline [--model llama-3-8b --quant q4f16_1 --requests 256]``
``torchrun --nproc-per-node N -m mlc_llm_b200.bench.decode_timeline``

After a warm-up pass it profiles twelve consecutive decode steps on rank 0 and prints (a) device time per
kernel and step, (b) one decode step in launch order with each kernel's duration and the gap to the
previous kernel.  The numbers are kernel durations inside CUDA-graph replays, not benchmark values.
"""

from __future__ import annotations

import argparse
import sys
import time

import numpy as np
import torch

from .. import parallel
from ..serve.config import EngineConfig


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--quant", default="q4f16_1")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--output-len", type=int, default=48)
    ap.add_argument("--out", default="")
    ap.add_argument("--model-args", default="", help='appended to the model string, e.g. "&expert_parallel=true"')
    args = ap.parse_args(argv)
    rank, world, local = parallel.env_world()
    comm = parallel.Communicator(tp_size=world, pp_size=1) if world > 1 else None
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    model = f"random://{args.model}?quant={args.quant}&seed=0{args.model_args}"
    r, p, o = args.requests, args.prompt_len, args.output_len
    cfg = EngineConfig(mode="server", max_num_sequence=r, prefill_chunk_size=8192,
                       max_total_sequence_length=r * (p + o) + 16 * r + 8192, prefix_cache_mode="disable",
                       gpu_memory_utilization=0.90)
    if rank != 0:
        from ..serve.engine_base import EngineRuntime  # pylint: disable=import-outside-toplevel

        cfg.model = model
        rt = EngineRuntime(cfg, device, comm=comm)
        for _ in range(2):
            comm.barrier()
            parallel.worker_loop(rt.executor, comm)
            torch.cuda.synchronize()
            comm.barrier()
        comm.destroy()
        return 0
    from ..serve.sync_engine import SyncMLCEngine  # pylint: disable=import-outside-toplevel

    eng = SyncMLCEngine(model, device, engine_config=cfg, comm=comm)
    rng = np.random.default_rng(1)
    gen = {"max_tokens": o, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
    lines = []

    def run(profile: bool) -> None:
        if comm is not None:
            comm.barrier()
        for i in range(r):
            eng.add_request(f"r{time.time()}-{i}", [rng.integers(0, 32000, p).tolist()], gen)
        n, prof = 0, None
        while not eng.empty():
            if profile and n == 30:
                prof = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA])
                prof.__enter__()
            eng.step()
            eng.take_outputs()
            n += 1
            if prof is not None and n == 42:
                torch.cuda.synchronize()
                prof.__exit__(None, None, None)
                rows = sorted(((e.key[:90], e.count, e.device_time_total) for e in prof.key_averages()),
                              key=lambda x: -x[2])
                total = sum(x[2] for x in rows)
                lines.append(f"12 decode steps on rank 0 of {world}: device time {total / 12 / 1000:.3f} ms per step")
                for k, c, t in rows[:16]:
                    if t > 0:
                        lines.append(f"{t / 12:9.1f} us/step {c / 12:6.1f} calls/step {t / max(c, 1):8.1f} us each  {k}")
                evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                             key=lambda e: e.time_range.start)
                start = next(i for i, e in enumerate(evs) if "embed" in e.name)
                lines.append("--- one decode step in launch order: start us, duration us, gap to the previous end us, kernel")
                prev = None
                for e in evs[start:start + 24]:
                    t0, t1 = e.time_range.start, e.time_range.end
                    lines.append(f"{t0 - evs[start].time_range.start:9.1f} {t1 - t0:8.1f} "
                                 f"{0 if prev is None else t0 - prev:7.1f}  {e.name[:70]}")
                    prev = t1
                prof = None
        torch.cuda.synchronize()
        if comm is not None:
            comm.shutdown_workers()
            comm.barrier()

    run(False)
    run(True)
    text = "\n".join(lines)
    print(text)
    if args.out:
        with open(args.out, "w", encoding="utf-8") as f:
            f.write(text + "\n")
    if comm is not None:
        comm.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
