"""Tensor parallelism over CPU ranks (gloo): sharded weights + step broadcast + worker loop must
reproduce the single-process result exactly (fp32)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


_SINGLE = {}


def _run(world: int, model: str, device: str = "cpu", port: int = 29531, extra_env=None, want_flags=False, timeout=600):
    # single-rank baselines repeat across tests: run each (model, device, settings) once
    key = (model, device, tuple(sorted((extra_env or {}).items())))
    if world == 1 and not want_flags:
        if key not in _SINGLE:
            _SINGLE[key] = _run_ranks(1, model, device, port, extra_env, False, timeout)
        return _SINGLE[key]
    return _run_ranks(world, model, device, port, extra_env, want_flags, timeout)


def _run_ranks(world: int, model: str, device: str, port: int, extra_env, want_flags, timeout):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_worker.py"),
           model, device]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    env.update(extra_env or {})
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    if out.returncode != 0:
        # keep the children's full stderr where a GPU run can pick it up
        log_dir = os.environ.get("MLCB_TEST_LOG_DIR", "")
        if log_dir and os.path.isdir(log_dir):
            with open(os.path.join(log_dir, "dist_stderr.log"), "w", encoding="utf-8") as f:
                f.write(out.stderr)
    assert out.returncode == 0, out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1]
    result = json.loads(line[len("RESULT "):])
    if want_flags:
        flags = [l for l in out.stdout.splitlines() if l.startswith("FLAGS ")][-1]
        return result, json.loads(flags[len("FLAGS "):])
    return result


@pytest.mark.parametrize("model", ["random://tiny-llama?quant=q0f32&seed=5",
                                   # latent attention with its heads split over the ranks + sharded experts
                                   "random://tiny-deepseek-v2?quant=q0f32&seed=5"])
def test_tp2_matches_single_rank(model):
    single = _run(1, model, port=29541)
    tp2 = _run(2, model, port=29542)
    assert single == tp2


def test_pp2_matches_single_rank():
    """Two pipeline stages over gloo p2p: stage 0 sends the hidden state on, the last stage returns
    the logits to rank 0; greedy tokens equal the single-process run exactly (fp32)."""
    model = "random://tiny-llama?quant=q0f32&seed=5"
    single = _run(1, model, port=29543)
    pp2 = _run(2, model, port=29544, extra_env={"MLCB_TEST_PP": "2"})
    assert single == pp2


def test_pp2_parallel_samples_keep_their_copied_pages():
    """``n = 2`` over two pipeline stages: the first decode step is offered to the deferred-read path, which a
    pipeline declines; the copy-on-write page copies of the forks that rode on that discarded plan must reach
    the model with the next one (prompt lengths 40, 9 and 23 all leave a partial last page)."""
    model = "random://tiny-llama?quant=q0f32&seed=5"
    single = _run(1, model, port=29563, extra_env={"MLCB_TEST_N": "2"})
    pp2 = _run(2, model, port=29564, extra_env={"MLCB_TEST_PP": "2", "MLCB_TEST_N": "2"})
    assert single == pp2
    assert all(s[0] == s[1] for s in single)  # greedy samples of one prompt are equal


def test_pp2_micro_batches_match_single_rank():
    """The same with prefill steps cut into two micro-batches (the threshold lowered so the short test prompts
    qualify): stage 1 works on the first half while stage 0 computes the second, the last stage returns the
    logit rows of both halves in one message; tokens stay exactly those of the single-process run."""
    model = "random://tiny-llama?quant=q0f32&seed=5"
    single = _run(1, model, port=29545)
    pp2, flags = _run(2, model, port=29546, extra_env={"MLCB_TEST_PP": "2", "MLCB_PP_MICROBATCH_MIN_TOKENS": "16"},
                      want_flags=True)
    assert single == pp2
    assert flags["pp_microbatch_steps"] >= 1


@pytest.mark.parametrize("model", ["random://tiny-rwkv5?quant=q0f32&seed=5", "random://tiny-rwkv6?quant=q0f32&seed=5",
                                   "random://tiny-qwen35?quant=q0f32&seed=5"])
def test_tp2_recurrent_model_matches_single_rank(model):
    """RWKV over two ranks: whole heads of the time-mix block (projections, decay, bonus, group norm, matrix
    state) and half the channel-mix width per rank; the workers find a sequence's state by the broadcast ids.
    Qwen3.5: key and value heads of the gated delta-rule layers (projection rows, convolution channels, decay
    parameters, state) and the gated attention heads are split the same way."""
    single = _run(1, model, port=29549)
    tp2 = _run(2, model, port=29550)
    assert single == tp2


def test_tp2_recurrent_model_with_parallel_samples():
    """``n = 2`` on two ranks: the fork pairs travel with the step descriptor, so the worker rank copies the
    state of the sequence its samples continue from as rank 0 does."""
    model = "random://tiny-rwkv6?quant=q0f32&seed=5"
    single = _run(1, model, port=29565, extra_env={"MLCB_TEST_N": "2"})
    tp2 = _run(2, model, port=29566, extra_env={"MLCB_TEST_N": "2"})
    assert single == tp2 and all(s[0] == s[1] for s in single)


@pytest.mark.parametrize("mode,head", [("eagle", "random://tiny-eagle?quant=q0f32&seed=3"),
                                       ("medusa", "random://tiny-medusa?quant=q0f32&seed=4")])
def test_tp2_with_a_feature_fed_draft_head_matches_plain_decoding(mode, head):
    """EAGLE: every rank runs its shard of the draft layer on feature rows that rank 0 sends; Medusa: rank 0
    evaluates the heads alone. Greedy speculative output is the plain single-process output."""
    model = "random://tiny-llama?quant=q0f32&seed=5"
    single = _run(1, model, port=29547)
    tp2, flags = _run(2, model, port=29548, extra_env={"MLCB_TEST_SPEC": f"{mode}={head}"}, want_flags=True)
    assert single == tp2
    assert flags["num_verify_steps"] > 0
