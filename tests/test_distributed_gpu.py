"""Tensor parallelism over NCCL on two GPUs: same greedy tokens as one GPU (up to fp16 noise)."""
import numpy as np
import pytest
import torch

from test_distributed_cpu import _run

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_nccl_matches_single_gpu():
    model = "random://tiny-llama-gpu?quant=q4f16_1&seed=5"
    single = _run(1, model, "cuda", port=29551)
    tp2 = _run(2, model, "cuda", port=29552)
    agree = np.mean([np.mean(np.asarray(a) == np.asarray(b)) for a, b in zip(single, tp2)])
    assert agree >= 0.7, (single, tp2)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("quant", ["q4f16_1", "q0f16"])
def test_tp2_fused_collectives_match_nccl_path(quant):
    """The fused GEMM+reduce-scatter / all-gather+GEMM kernels over peer memory against the same
    model on the NCCL all-reduce path."""
    model = f"random://tiny-llama-gpu?quant={quant}&seed=5"
    env = {"NCCL_NVLS_ENABLE": "0"}
    nccl, f0 = _run(2, model, "cuda", port=29553, extra_env=dict(env, MLCB_FUSED_TP="0"), want_flags=True)
    fused, f1 = _run(2, model, "cuda", port=29554, extra_env=dict(env, MLCB_FUSED_TP="1"), want_flags=True)
    assert not f0["fused_tp"] and f1["fused_tp"] and f1["fused_launches"] > 0
    agree = np.mean([np.mean(np.asarray(a) == np.asarray(b)) for a, b in zip(nccl, fused)])
    assert agree >= 0.7, (nccl, fused)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_fused_forward_replayed_from_cuda_graphs():
    """Both ranks capture the fused forward of a decode shape and replay it; the kernels' call numbers
    come from device memory, so the replays exchange rows exactly like the eager launches do."""
    model = "random://tiny-llama-gpu?quant=q4f16_1&seed=5"
    env = {"NCCL_NVLS_ENABLE": "0", "MLCB_FUSED_TP": "1"}
    eager, f0 = _run(2, model, "cuda", port=29559, extra_env=dict(env, MLCB_CUDA_GRAPH="0"), want_flags=True,
                     timeout=180)
    graph, f1 = _run(2, model, "cuda", port=29560, extra_env=dict(env, MLCB_CUDA_GRAPH="1"), want_flags=True,
                     timeout=180)
    assert f0["graph_replays"] == 0 and f1["graph_replays"] > 0 and f1["fused_tp"]
    agree = np.mean([np.mean(np.asarray(a) == np.asarray(b)) for a, b in zip(eager, graph)])
    assert agree >= 0.9, (eager, graph)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep2_all_to_all_matches_tensor_parallel_moe():
    """Mixtral-style MoE with experts distributed over the ranks (all-to-all dispatch / combine over
    peer memory) against the same model with width-sharded experts and NCCL all-reduce."""
    env = {"NCCL_NVLS_ENABLE": "0", "MLCB_FUSED_TP": "0"}
    base = "random://tiny-mixtral-gpu?quant=q0f16&seed=7"
    tp = _run(2, base, "cuda", port=29555, extra_env=env)
    ep = _run(2, base + "&expert_parallel=true", "cuda", port=29556, extra_env=env)
    agree = np.mean([np.mean(np.asarray(a) == np.asarray(b)) for a, b in zip(tp, ep)])
    assert agree >= 0.7, (tp, ep)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pp2_nccl_p2p_matches_single_gpu():
    """Two pipeline stages on two GPUs: hidden states and logits travel over NCCL send / recv."""
    model = "random://tiny-llama-gpu?quant=q0f16&seed=5"
    single = _run(1, model, "cuda", port=29557)
    pp2 = _run(2, model, "cuda", port=29558, extra_env={"MLCB_TEST_PP": "2", "NCCL_NVLS_ENABLE": "0"})
    agree = np.mean([np.mean(np.asarray(a) == np.asarray(b)) for a, b in zip(single, pp2)])
    assert agree >= 0.9, (single, pp2)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_eagle_head_runs_sharded_and_keeps_the_greedy_output():
    """Two ranks, fused tensor-parallel target + an EAGLE head whose layer is sharded the same way: rank 0 sends
    the feature rows of every draft call to rank 1. Greedy tokens stay those of plain TP2 decoding (a near-tie
    between the verification batch and the one-token step may move a late token in fp16)."""
    model = "random://tiny-llama-tp8?quant=q0f16&seed=5"
    plain = _run(2, model, "cuda", port=29571)
    spec, flags = _run(2, model, "cuda", port=29572, want_flags=True,
                       extra_env={"MLCB_TEST_SPEC": "eagle=random://tiny-eagle-tp8?quant=q0f16&seed=3"})
    assert flags["num_verify_steps"] > 0
    same = sum(int(a == b) for p, s in zip(plain, spec) for a, b in zip(p, s))
    total = sum(len(p) for p in plain)
    assert [p[0] for p in plain] == [s[0] for s in spec] and same >= 0.5 * total, (plain, spec)
