"""``python -m mlc_llm_b200.bench`` / ``python -m mlc_llm_b200 bench``: HTTP load generator (reference:
``python/mlc_llm/bench/__main__.py:129-403``)."""

from __future__ import annotations

import argparse
import json
import random
from typing import List, Optional

import numpy as np
import requests

from ..tokenizers import Tokenizer
from .api_endpoint import SUPPORTED_BACKENDS, create_api_endpoint
from .dataset import SUPPORTED_DATASET, create_dataset
from .request_processor import MetricAnalyzer, create_pipelines
from .request_record import convert_reports_to_df, generate_metrics_summary, pretty_print_report


def _ints(text: Optional[str]) -> Optional[List[int]]:
    return None if text is None else [int(x) for x in text.split(",")]


def _floats(text: Optional[str]) -> Optional[List[float]]:
    if text is None:
        return None
    vals = [float(x) for x in text.split(",")]
    if any(v <= 0 for v in vals):
        raise argparse.ArgumentTypeError("request rates must be positive")
    return vals


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("mlc_llm_b200 bench")
    p.add_argument("--dataset", type=str, choices=SUPPORTED_DATASET, default=None)
    p.add_argument("--dataset-path", type=str, default=None)
    p.add_argument("--api-endpoint", type=str, choices=SUPPORTED_BACKENDS, default="openai")
    p.add_argument("--tokenizer", type=str, required=True, help="model directory holding the tokenizer")
    p.add_argument("--model", type=str, default=None, help="model name sent in requests (default: --tokenizer)")
    p.add_argument("--num-gpus", type=int, required=True)
    p.add_argument("--num-requests", type=int, required=True)
    p.add_argument("--num-warmup-requests", type=int, default=0)
    p.add_argument("--per-gpu-workload", action="store_true")
    p.add_argument("--num-concurrent-requests", type=_ints, default=None)
    p.add_argument("--request-rate", type=_floats, default=None)
    p.add_argument("--replay-timestamp-scale", type=float, default=None)
    p.add_argument("--input-len", type=int, default=None)
    p.add_argument("--input-len-std", type=float, default=0)
    p.add_argument("--output-len", type=int, default=None)
    p.add_argument("--output-len-std", type=float, default=0)
    p.add_argument("--stream", action="store_true", default=True)
    p.add_argument("--include-server-metrics", action="store_true")
    p.add_argument("--host", type=str, required=True)
    p.add_argument("--port", type=int, required=True)
    p.add_argument("--timeout", type=float, default=3 * 60 * 60)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--apply-chat-template", action="store_true")
    p.add_argument("--loogle-task", type=str, default="shortdep_qa",
                   help="LooGLE test set: shortdep_qa, longdep_qa, longdep_summarization or shortdep_cloze")
    p.add_argument("--num-process-workers", type=int, default=None)
    p.add_argument("--disable-tqdm", action="store_true")
    p.add_argument("--max-schedule-gap", type=float, default=0.5)
    p.add_argument("--mlc-model-lib", type=str, default=None)
    p.add_argument("--mlc-engine-config", type=str, default=None)
    p.add_argument("--cuda-profile", action="store_true")
    p.add_argument("--debug-dump", action="store_true")
    p.add_argument("--multi-round", action="store_true")
    p.add_argument("--output", "-o", type=str, default="mlc_benchmark.csv")
    return p


def _load_tokenizer(path: str) -> Tokenizer:
    try:
        return Tokenizer(path)
    except (ValueError, FileNotFoundError):
        return Tokenizer.synthetic(32000)


def run(args) -> List[dict]:
    random.seed(args.seed)
    np.random.seed(args.seed)
    tokenizer = _load_tokenizer(args.tokenizer)
    dataset = create_dataset(args, tokenizer)
    pipelines = create_pipelines(args, lambda: create_api_endpoint(args), dataset)
    reports = []
    total = args.num_requests * (args.num_gpus if args.per_gpu_workload else 1)
    for pipeline in pipelines:
        records = dataset.generate_request_records(args.input_len, args.output_len, args.input_len_std,
                                                   args.output_len_std)
        if args.cuda_profile:
            requests.post(f"http://{args.host}:{args.port}/debug/cuda_profiler_start", timeout=10)
        records = pipeline(records)
        if args.cuda_profile:
            requests.post(f"http://{args.host}:{args.port}/debug/cuda_profiler_stop", timeout=10)
        records = MetricAnalyzer(tokenizer)(records)
        report = generate_metrics_summary(records, total, args.num_gpus)
        pretty_print_report(report)
        if args.debug_dump:
            with open(args.output + ".records.jsonl", "a", encoding="utf-8") as f:
                for r in records:
                    f.write(json.dumps({"id": r.request_id, "output": r.output_str, "error": r.error_msg}) + "\n")
        reports.append(report)
        try:
            r = requests.post(f"http://{args.host}:{args.port}/debug/dump_engine_metrics", json={}, timeout=10)
            if r.status_code == 200 and args.include_server_metrics:
                report["engine_metrics"] = r.json()
        except requests.RequestException:
            pass
    convert_reports_to_df([{k: v for k, v in r.items() if k != "engine_metrics"} for r in reports]
                          ).to_csv(args.output, index=False)
    return reports


def main(argv=None) -> None:
    run(build_parser().parse_args(argv))


if __name__ == "__main__":
    main()
