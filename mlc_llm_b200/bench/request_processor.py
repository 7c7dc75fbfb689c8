"""Workload pipelines of the load generator (reference: ``python/mlc_llm/bench/request_processor.py``):
sampling, sampling-option attachment, warm-up, the executors (fixed concurrency, fixed request rate /
timestamp replay) and the metric analyser."""

from __future__ import annotations

import asyncio
import copy
import random
import time
from typing import Callable, List, Optional

import numpy as np

from .api_endpoint import APIEndPoint
from .request_record import RequestRecord


class RequestProcessor:
    def __call__(self, records: List[RequestRecord]) -> List[RequestRecord]:
        raise NotImplementedError


def _each(records):
    """Every record that is sent: plain ones and the members of groups."""
    for r in records:
        members = getattr(r, "records", None)
        if members is None:
            yield r
        else:
            yield from members


class SampleRequests(RequestProcessor):
    def __init__(self, num_requests: int, take_first_x_requests: bool = False):
        self.n, self.first = num_requests, take_first_x_requests

    def __call__(self, records):
        if len(records) < self.n:
            # recycle when the dataset is smaller than the run
            records = [records[i % len(records)] for i in range(self.n)]
            records = [copy.deepcopy(r) for r in records]
        elif self.first:
            records = records[: self.n]
        else:
            records = random.sample(records, self.n)
        for i, r in enumerate(records):
            r.request_id = i
        return records


class AttachModelName(RequestProcessor):
    def __init__(self, model: str):
        self.model = model

    def __call__(self, records):
        for r in _each(records):
            r.chat_cmpl["model"] = self.model
        return records


class AttachSamplingOptions(RequestProcessor):
    def __init__(self, temperature: float, top_p: float, ignore_eos: bool):
        self.t, self.p, self.ignore_eos = temperature, top_p, ignore_eos

    def __call__(self, records):
        for r in _each(records):
            r.chat_cmpl["temperature"] = self.t
            r.chat_cmpl["top_p"] = self.p
            r.chat_cmpl.setdefault("frequency_penalty", 0.0)
            r.chat_cmpl.setdefault("presence_penalty", 0.0)
            if self.ignore_eos:
                r.chat_cmpl["debug_config"] = dict(r.chat_cmpl.get("debug_config") or {}, ignore_eos=True)
        return records


class AttachRequestRateTimestamp(RequestProcessor):
    """Poisson arrivals at ``request_rate`` per second."""

    def __init__(self, request_rate: float):
        self.rate = float(request_rate)

    def __call__(self, records):
        t = 0.0
        for r in records:
            t += float(np.random.exponential(1.0 / self.rate))
            r.timestamp = t
        return records


class ScaleTimestamp(RequestProcessor):
    def __init__(self, scale: Optional[float]):
        self.scale = scale

    def __call__(self, records):
        if self.scale is not None:
            for r in records:
                if r.timestamp is not None:
                    r.timestamp *= self.scale
        return records


class MetricAnalyzer(RequestProcessor):
    """Fills the token counts the server did not report (with the tokenizer) and derives TPOT / ITL:
    TPOT = (e2e - TTFT) / (output tokens - tokens in the first chunk); ITL = e2e / output tokens."""

    def __init__(self, tokenizer):
        self.tok = tokenizer

    def __call__(self, records):
        out = []
        for r in records:
            m = r.metrics
            if m is None or not m.success:
                out.append(r)
                continue
            if m.output_tokens is None:
                m.output_tokens = len(self.tok.encode(r.output_str or ""))
            if m.input_tokens is None:
                if r.input_token_ids is not None:
                    m.input_tokens = len(r.input_token_ids)
                else:
                    m.input_tokens = sum(len(self.tok.encode(x.get("content") or ""))
                                         for x in r.chat_cmpl.get("messages", []))
            first = len(self.tok.encode(r.first_chunk_output_str)) if r.first_chunk_output_str else 1
            if m.output_tokens <= 0 or m.time_to_first_token_s is None:
                m.success = False
                r.error_msg = r.error_msg or "no output tokens"
                out.append(r)
                continue
            m.inter_token_latency_s = m.end_to_end_latency_s / m.output_tokens
            denom = m.output_tokens - first
            m.time_per_output_token_s = (m.end_to_end_latency_s - m.time_to_first_token_s) / denom if denom > 0 else 0.0
            out.append(r)
        return out


class Executor(RequestProcessor):
    def __init__(self, make_endpoint: Callable[[], APIEndPoint], disable_tqdm: bool = True):
        self.make_endpoint = make_endpoint
        self.disable_tqdm = disable_tqdm


async def _send(ep, rec) -> List[RequestRecord]:
    """One record through the endpoint; the members of a group go in order, one at a time."""
    members = getattr(rec, "records", None)
    if members is None:
        return [await ep(rec)]
    out = []
    for m in members:
        if m.timestamp is None:
            m.timestamp = rec.timestamp
        out.append(await ep(m))
    return out


class FixedConcurrentRequestExecutor(Executor):
    """Keeps ``num_concurrent`` requests in flight until the workload is exhausted."""

    def __init__(self, make_endpoint, num_concurrent: int, disable_tqdm: bool = True):
        super().__init__(make_endpoint, disable_tqdm)
        self.n = num_concurrent

    def __call__(self, records):
        async def run():
            queue = list(reversed(records))
            done: List[RequestRecord] = []
            async with self.make_endpoint() as ep:
                async def worker():
                    while queue:
                        rec = queue.pop()
                        done.extend(await _send(ep, rec))

                await asyncio.gather(*[worker() for _ in range(min(self.n, len(records)))])
            return done

        return asyncio.run(run())


class FixTimestampExecutor(Executor):
    """Sends each request at its timestamp (request-rate mode and trace replay)."""

    def __init__(self, make_endpoint, max_schedule_gap: float = 0.5, disable_tqdm: bool = True):
        super().__init__(make_endpoint, disable_tqdm)
        self.gap = max_schedule_gap

    def __call__(self, records):
        async def run():
            async with self.make_endpoint() as ep:
                t0 = time.monotonic()

                async def fire(rec):
                    delay = (rec.timestamp or 0.0) - (time.monotonic() - t0)
                    if delay > 0:
                        await asyncio.sleep(delay)
                    return await _send(ep, rec)

                return [r for group in await asyncio.gather(*[fire(r) for r in records]) for r in group]

        return asyncio.run(run())


class WarmupAndRun(RequestProcessor):
    """Runs the first ``num_warmup`` records untimed, then the rest."""

    def __init__(self, num_warmup: int, num_benchmark: int, pipeline: RequestProcessor):
        self.nw, self.nb, self.pipeline = num_warmup, num_benchmark, pipeline

    def __call__(self, records):
        warm, bench = records[: self.nw], records[self.nw: self.nw + self.nb]
        if warm:
            self.pipeline(warm)
        for i, r in enumerate(bench):
            r.request_id = i
        return self.pipeline(bench)


class SequentialProcessor(RequestProcessor):
    def __init__(self, *stages: RequestProcessor):
        self.stages = stages

    def __call__(self, records):
        for s in self.stages:
            records = s(records)
        return records


def create_pipelines(args, make_endpoint, dataset) -> List[RequestProcessor]:
    """One pipeline per requested concurrency / request rate (or a single timestamp replay)."""
    total = args.num_requests * (args.num_gpus if args.per_gpu_workload else 1)
    common = [SampleRequests(total + args.num_warmup_requests),
              AttachModelName(args.model or args.tokenizer),
              AttachSamplingOptions(args.temperature, args.top_p, args.ignore_eos)]
    pipelines: List[RequestProcessor] = []
    if args.num_concurrent_requests:
        for n in args.num_concurrent_requests:
            n_total = n * (args.num_gpus if args.per_gpu_workload else 1)
            pipelines.append(SequentialProcessor(
                *common, WarmupAndRun(args.num_warmup_requests, total,
                                      FixedConcurrentRequestExecutor(make_endpoint, n_total, args.disable_tqdm))))
    elif args.request_rate:
        for rate in args.request_rate:
            rate_total = rate * (args.num_gpus if args.per_gpu_workload else 1)
            pipelines.append(SequentialProcessor(
                *common, AttachRequestRateTimestamp(rate_total),
                WarmupAndRun(args.num_warmup_requests, total,
                             FixTimestampExecutor(make_endpoint, args.max_schedule_gap, args.disable_tqdm))))
    else:
        if not dataset.timestamp_available:
            raise ValueError("give --num-concurrent-requests or --request-rate (this dataset has no timestamps)")
        pipelines.append(SequentialProcessor(
            *common, ScaleTimestamp(args.replay_timestamp_scale),
            WarmupAndRun(args.num_warmup_requests, total,
                         FixTimestampExecutor(make_endpoint, args.max_schedule_gap, args.disable_tqdm))))
    return pipelines
