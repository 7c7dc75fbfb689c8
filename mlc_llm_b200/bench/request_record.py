"""Per-request records and the summary statistics of a load-generator run (reference:
``python/mlc_llm/bench/request_record.py:15-200``)."""

from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

import numpy as np


@dataclasses.dataclass
class ServerMetrics:
    input_tokens: int = 0
    prefill_tokens: int = 0
    output_tokens: int = 0
    end_to_end_latency_s: float = 0.0
    prefill_tokens_per_s: float = 0.0
    inter_token_latency_s: float = 0.0
    time_per_output_token_s: float = 0.0
    time_to_first_token_s: Optional[float] = None


@dataclasses.dataclass
class Metrics:
    success: bool = False
    start_time: float = 0.0
    finish_time: float = 0.0
    end_to_end_latency_s: float = 0.0
    input_tokens: Optional[int] = None
    output_tokens: Optional[int] = None
    inter_token_latency_s: Optional[float] = None
    time_per_output_token_s: Optional[float] = None
    time_to_first_token_s: Optional[float] = None
    server_metrics: Optional[ServerMetrics] = None
    exec_feature: Optional[Dict[str, Any]] = None


@dataclasses.dataclass
class RequestRecord:
    """One request of the workload: the chat-completion body to send, what came back, its timings."""

    request_id: Optional[int] = None
    chat_cmpl: Dict[str, Any] = dataclasses.field(default_factory=dict)
    output_str: Optional[str] = None
    first_chunk_output_str: str = ""
    timestamp: Optional[float] = None
    metrics: Optional[Metrics] = None
    error_msg: Optional[str] = None
    input_token_ids: Optional[List[int]] = None  # token-id prompts go to /v1/completions


@dataclasses.dataclass
class GroupedRequestRecord(RequestRecord):
    """Requests that belong together (the questions on one long document, the turns of one agent trace):
    an executor sends them one after the other from the same worker, so each can reuse the KV prefix the
    previous one left in the server (reference: ``GroupedRequestRecord``, ``bench/request_record.py``)."""

    records: List[RequestRecord] = dataclasses.field(default_factory=list)


_QUANTILES = (25, 50, 75, 90, 95, 99)


def _stats(values: List[float]) -> Dict[str, float]:
    if not values:
        return {}
    a = np.asarray(values, dtype=np.float64)
    out = {"quantiles": {f"p{q}": float(np.percentile(a, q)) for q in _QUANTILES},
           "mean": float(a.mean()), "min": float(a.min()), "max": float(a.max()), "stddev": float(a.std())}
    return out


def generate_metrics_summary(records: List[RequestRecord], num_total_requests: int, num_gpus: int
                             ) -> Dict[str, Any]:
    """Throughputs over the whole run (sum of tokens / (last finish - first start)) and the
    distribution of every per-request latency metric."""
    ok = [r for r in records if r.metrics is not None and r.metrics.success]
    report: Dict[str, Any] = {"num_gpus": num_gpus, "num_total_requests": num_total_requests,
                              "num_completed_requests": len(ok), "num_failed_requests": len(records) - len(ok)}
    if not ok:
        return report
    start = min(r.metrics.start_time for r in ok)
    finish = max(r.metrics.finish_time for r in ok)
    span = max(finish - start, 1e-9)
    in_tok = sum(r.metrics.input_tokens or 0 for r in ok)
    out_tok = sum(r.metrics.output_tokens or 0 for r in ok)
    report.update({
        "request_throughput": len(ok) / span, "input_token_throughput": in_tok / span,
        "output_token_throughput": out_tok / span,
        "request_throughput_per_gpu": len(ok) / span / max(1, num_gpus),
        "input_token_throughput_per_gpu": in_tok / span / max(1, num_gpus),
        "output_token_throughput_per_gpu": out_tok / span / max(1, num_gpus),
        "duration_s": span,
    })
    for name in ("end_to_end_latency_s", "time_to_first_token_s", "time_per_output_token_s",
                 "inter_token_latency_s", "input_tokens", "output_tokens"):
        vals = [getattr(r.metrics, name) for r in ok if getattr(r.metrics, name) is not None]
        report[name] = _stats([float(v) for v in vals])
    server = [r.metrics.server_metrics for r in ok if r.metrics.server_metrics is not None]
    if server:
        report["server_metrics"] = {
            f.name: _stats([float(getattr(s, f.name)) for s in server if getattr(s, f.name) is not None])
            for f in dataclasses.fields(ServerMetrics)}
    return report


def pretty_print_report(report: Dict[str, Any]) -> str:
    lines = [f"{' Benchmark result ':=^60}"]

    def put(name, value):
        lines.append(f"{name:<44}{value:>16}")

    for key in ("num_gpus", "num_total_requests", "num_completed_requests", "num_failed_requests"):
        if key in report:
            put(key, report[key])
    for key in ("duration_s", "request_throughput", "input_token_throughput", "output_token_throughput",
                "output_token_throughput_per_gpu"):
        if key in report:
            put(key, f"{report[key]:.3f}")
    for key in ("time_to_first_token_s", "time_per_output_token_s", "inter_token_latency_s",
                "end_to_end_latency_s"):
        st = report.get(key)
        if st:
            lines.append(f"{' ' + key + ' ':-^60}")
            put("mean", f"{st['mean']:.4f}")
            for q, v in st["quantiles"].items():
                put(q, f"{v:.4f}")
    out = "\n".join(lines)
    print(out)
    return out


def convert_reports_to_df(reports: List[Dict[str, Any]]):
    """Flatten reports into one pandas row each (for the CSV the command writes)."""
    import pandas as pd  # pylint: disable=import-outside-toplevel

    def flatten(d, pre=""):
        out = {}
        for k, v in d.items():
            if isinstance(v, dict):
                out.update(flatten(v, f"{pre}{k}."))
            else:
                out[pre + k] = v
        return out

    return pd.DataFrame([flatten(r) for r in reports])
