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
