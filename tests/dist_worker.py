"""Child process of the multi-rank tests: runs a tiny model tensor-parallel (gloo on CPU, NCCL on
GPUs) and, on rank 0, prints the generated token ids as JSON."""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mlc_llm_b200 import parallel  # noqa: E402
from mlc_llm_b200.serve.config import EngineConfig  # noqa: E402
from mlc_llm_b200.serve.engine_base import EngineRuntime  # noqa: E402


def main():
    model = sys.argv[1]
    device = sys.argv[2]
    rank, world, local = parallel.env_world()
    dev = torch.device("cuda", local) if device == "cuda" else torch.device("cpu")
    pp = int(os.environ.get("MLCB_TEST_PP", "1"))
    comm = parallel.Communicator(tp_size=world // pp, pp_size=pp, device=dev,
                                 timeout_s=int(os.environ.get("MLCB_TEST_COMM_TIMEOUT_S", "120")))
    cfg = EngineConfig(model=model, mode="server", max_num_sequence=8, prefill_chunk_size=64,
                       max_total_sequence_length=1024, prefix_cache_mode="disable",
                       tensor_parallel_shards=world // pp, pipeline_parallel_stages=pp)
    spec = os.environ.get("MLCB_TEST_SPEC", "")
    if spec:  # "eagle=<model string>" / "medusa=<model string>": a feature-fed draft head beside the model
        cfg.speculative_mode, head = spec.split("=", 1)
        cfg.spec_draft_length = 3
        cfg.additional_models = [head]
    exit_after = int(os.environ.get("MLCB_TEST_WORKER_EXIT_AFTER", "0"))
    if rank != 0:
        rt = EngineRuntime(cfg, dev, comm=comm)
        if exit_after:
            # failure injection on the host: this rank leaves between two steps, with nothing in flight
            steps = {"n": 0}
            orig = rt.executor.worker_step

            def counted(*a, **k):
                out = orig(*a, **k)
                steps["n"] += 1
                if steps["n"] >= exit_after:
                    os._exit(0)
                return out

            rt.executor.worker_step = counted
        parallel.worker_loop(rt.executor, comm)
        comm.destroy()
        return
    from mlc_llm_b200.serve.sync_engine import SyncMLCEngine

    eng = SyncMLCEngine(model, dev, engine_config=cfg, comm=comm)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 32000, int(n)).tolist() for n in (40, 9, 23)]
    logits_out = os.environ.get("MLCB_TEST_LOGITS_OUT")
    captured = []
    if logits_out:
        # numerics runs: keep the logits of every sampling call (greedy sampling goes through ops.argmax);
        # prompts cross several 32-row chunks of the fused collectives, the last chunk uneven
        from mlc_llm_b200 import ops

        prompts = [rng.integers(0, 32000, int(n)).tolist() for n in (70, 33, 41)]
        orig_argmax = ops.argmax

        def keep(x):
            captured.append(x.detach().float().cpu().numpy())
            return orig_argmax(x)

        ops.argmax = keep
        zero = os.environ.get("MLCB_TEST_ZERO_SHARD")
        if zero:
            # oracle with one rank's contribution to a row-parallel projection removed (see the numerics tests)
            zw, zr = (int(v) for v in zero.split(","))
            lw = eng.runtime.models[0].p.linears["model.layers.0.self_attn.o_proj"]
            k = lw.w.shape[1]
            lw.w[:, zr * k // zw:(zr + 1) * k // zw] = 0
            lw._dense = None
    try:
        gen = {"max_tokens": 8, "temperature": 0.0, "debug_config": {"ignore_eos": True}}
        samples = int(os.environ.get("MLCB_TEST_N", "1"))
        if samples > 1:
            gen["n"] = samples  # parallel samples: forks with copy-on-write of the last partial page
        _, toks = eng.generate(prompts, gen)
    except Exception as err:  # pylint: disable=broad-except
        if not exit_after:
            raise
        print("FAILURE " + json.dumps({"rank": rank, "error": str(err)[:300]}), flush=True)
        os._exit(0)
    comm.shutdown_workers()
    if logits_out:
        np.savez(logits_out, *captured)
    rt = eng.runtime
    print("FLAGS " + json.dumps({"fused_tp": bool(getattr(rt, "fused_tp", False)),
                                 "graph_replays": int(rt.executor.graph_replays),
                                 "pp_microbatch_steps": int(rt.executor.pp_microbatch_steps),
                                 "num_verify_steps": int(json.loads(eng.debug_stats()).get("num_verify_steps", 0)),
                                 "fused_launches": int(rt.models[0].fused.launches) if getattr(rt.models[0], "fused", None) else 0}),
          flush=True)
    print("RESULT " + json.dumps([t[0] for t in toks] if samples == 1 else toks), flush=True)
    comm.destroy()


if __name__ == "__main__":
    main()
