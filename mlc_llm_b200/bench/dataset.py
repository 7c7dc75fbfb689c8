"""Workload sources of the load generator (reference: ``python/mlc_llm/bench/dataset.py``).

Every dataset produces :class:`RequestRecord` s holding an OpenAI chat-completion body.  Without
network access the file-based datasets need ``--dataset-path``; ``synthetic`` needs nothing."""

from __future__ import annotations

import json
import random
from typing import Any, Dict, List, Optional

import numpy as np

from .request_record import RequestRecord


class Dataset:
    """Base: subclasses fill ``self.requests`` with (prompt text or ids, suggested output length)."""

    require_fake_warmup = False
    timestamp_available = False

    def generate_request_records(self, input_len: Optional[int], output_len: Optional[int],
                                 input_len_std: float = 0.0, output_len_std: float = 0.0) -> List[RequestRecord]:
        raise NotImplementedError


def _len_sample(mean: Optional[int], std: float, default: int) -> int:
    if mean is None:
        return default
    if std <= 0:
        return int(mean)
    return max(1, int(round(np.random.normal(mean, std))))


class SyntheticDataset(Dataset):
    """Uniform-random token ids of the requested length (the serving benchmark's workload)."""

    def __init__(self, tokenizer, num_requests: int = 1000, vocab_size: Optional[int] = None):
        self.tokenizer = tokenizer
        self.num = num_requests
        self.vocab = vocab_size or getattr(tokenizer, "vocab_size", 32000)
        if callable(self.vocab):
            self.vocab = self.vocab()

    def generate_request_records(self, input_len, output_len, input_len_std=0.0, output_len_std=0.0):
        out = []
        for _ in range(self.num):
            n_in = _len_sample(input_len, input_len_std, 512)
            n_out = _len_sample(output_len, output_len_std, 128)
            ids = np.random.randint(10, max(11, int(self.vocab) - 10), size=n_in).tolist()
            out.append(RequestRecord(chat_cmpl={"messages": [], "max_tokens": n_out, "model": ""},
                                     input_token_ids=ids))
        return out


class TextPromptDataset(Dataset):
    """Prompts from a file, truncated / sampled to the requested lengths with the tokenizer."""

    def __init__(self, prompts: List[Dict[str, Any]], tokenizer, apply_chat_template: bool = False):
        self.prompts = prompts
        self.tokenizer = tokenizer
        self.apply_chat_template = apply_chat_template

    def generate_request_records(self, input_len, output_len, input_len_std=0.0, output_len_std=0.0):
        out = []
        for item in self.prompts:
            text = item["prompt"]
            ids = self.tokenizer.encode(text)
            if input_len is not None:
                want = _len_sample(input_len, input_len_std, len(ids))
                if len(ids) < want:
                    continue
                text = self.tokenizer.decode(ids[:want])
            n_out = _len_sample(output_len, output_len_std, item.get("output_len") or 128)
            body = {"messages": [{"role": "user", "content": text}], "max_tokens": n_out, "model": ""}
            if "response_format" in item:
                body["response_format"] = item["response_format"]
            out.append(RequestRecord(chat_cmpl=body, timestamp=item.get("timestamp")))
        return out


def _load_sharegpt(path: str, tokenizer) -> List[Dict[str, Any]]:
    with open(path, encoding="utf-8") as f:
        raw = json.load(f)
    prompts = []
    for conv in raw:
        turns = conv.get("conversations", [])
        if len(turns) < 2 or turns[0].get("from") != "human":
            continue
        out_len = len(tokenizer.encode(turns[1]["value"]))
        if out_len < 4:
            continue
        prompts.append({"prompt": turns[0]["value"], "output_len": out_len})
    random.shuffle(prompts)
    return prompts


def _load_jsonl_prompts(path: str, key: str = "prompt") -> List[Dict[str, Any]]:
    prompts = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                d = json.loads(line)
                prompts.append({"prompt": d[key], "output_len": d.get("output_len"),
                                "timestamp": d.get("timestamp")})
    return prompts


def _load_json_mode_eval(path: str) -> List[Dict[str, Any]]:
    with open(path, encoding="utf-8") as f:
        raw = json.load(f)
    prompts = []
    for item in raw:
        schema = item.get("schema")
        prompts.append({"prompt": item["prompt"],
                        "response_format": {"type": "json_object",
                                            "schema": json.dumps(schema) if not isinstance(schema, str) else schema}})
    return prompts


SUPPORTED_DATASET = ["synthetic", "sharegpt", "llmperf", "json-mode-eval", "loogle", "react", "wildchat",
                     "azure-llm-inference"]


def create_dataset(args, tokenizer) -> Dataset:
    name = args.dataset or ("synthetic" if args.dataset_path is None else "sharegpt")
    if name == "synthetic":
        return SyntheticDataset(tokenizer, args.num_requests + args.num_warmup_requests)
    if args.dataset_path is None:
        raise ValueError(f"dataset {name!r} needs --dataset-path (no network access to fetch it)")
    if name == "sharegpt":
        return TextPromptDataset(_load_sharegpt(args.dataset_path, tokenizer), tokenizer, args.apply_chat_template)
    if name == "json-mode-eval":
        return TextPromptDataset(_load_json_mode_eval(args.dataset_path), tokenizer)
    ds = TextPromptDataset(_load_jsonl_prompts(args.dataset_path), tokenizer, args.apply_chat_template)
    if name == "azure-llm-inference":
        ds.timestamp_available = True
    return ds
