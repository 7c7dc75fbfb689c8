"""Command line of ``mlc_llm_b200 calibrate`` (reference: ``python/mlc_llm/cli/calibrate.py``)."""

from __future__ import annotations

import argparse

from ..interface.calibrate import calibrate
from .serve import EngineConfigOverride


def main(argv) -> None:
    p = argparse.ArgumentParser("mlc_llm_b200 calibrate",
                                description="Record activation ranges of every linear layer on a dataset")
    p.add_argument("model", type=str, help="model directory (with mlc-chat-config.json), or random://<preset>")
    p.add_argument("--device", type=str, default="auto")
    p.add_argument("--model-lib", type=str, default=None, help="accepted for command-line compatibility")
    p.add_argument("--output", "-o", type=str, required=True,
                   help="tensor-cache directory that receives the calibration scales (updated in place)")
    p.add_argument("--dataset", type=str, required=True,
                   help="ShareGPT-format JSON: a list of {conversations: [{value}, {value}, ...]}")
    p.add_argument("--num-calibration-samples", type=int, default=16)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--overrides", type=EngineConfigOverride.from_str, default="")
    a = p.parse_args(argv)
    o = a.overrides
    stats = calibrate(model=a.model, device=a.device, model_lib=a.model_lib, dataset=a.dataset, output=a.output,
                      num_calibration_samples=a.num_calibration_samples, seed=a.seed,
                      max_num_sequence=o.max_num_sequence, max_total_sequence_length=o.max_total_seq_length,
                      prefill_chunk_size=o.prefill_chunk_size, max_history_size=o.max_history_size,
                      gpu_memory_utilization=o.gpu_memory_utilization)
    print(f"calibrated {len(stats)} linear layers -> {a.output}")
