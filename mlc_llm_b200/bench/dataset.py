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


def _user(text: str, max_tokens: int, **extra) -> Dict[str, Any]:
    return dict({"messages": [{"role": "user", "content": text}], "max_tokens": int(max_tokens), "model": ""},
                **extra)


def _records_of(path: str) -> List[Dict[str, Any]]:
    """A ``.json`` file holding a list, or a ``.jsonl`` file with one object per line."""
    with open(path, encoding="utf-8") as f:
        if path.endswith(".jsonl"):
            return [json.loads(line) for line in f if line.strip()]
        data = json.load(f)
    return data if isinstance(data, list) else data.get("data", [])


class LLMPerfDataset(Dataset):
    """Prompts of a requested token length assembled from the shuffled lines of a text file (the reference
    uses a sonnet file): an instruction line followed by lines until the length is reached, the last one cut
    at the token boundary. Requests ignore EOS so the output length is exact.
    Reference behaviour: ``LLMPerfDataset`` (``python/mlc_llm/bench/dataset.py:262-340``)."""

    def __init__(self, path: str, num_requests: int, tokenizer):
        self.tokenizer, self.num = tokenizer, num_requests
        with open(path, encoding="utf-8") as f:
            self.lines = [ln for ln in f.readlines() if ln.strip()]
        if not self.lines:
            raise ValueError(f"{path}: no text lines")
        self.line_ids = [tokenizer.encode(ln) for ln in self.lines]

    def generate_request_records(self, input_len=None, output_len=None, input_len_std=250.0, output_len_std=0.0):
        input_len = 550 if input_len is None or input_len < 40 else input_len
        output_len = 150 if output_len is None else output_len
        out = []
        order = list(range(len(self.lines)))
        for _ in range(self.num):
            n_in = max(8, _len_sample(input_len, input_len_std, input_len))
            n_out = max(1, _len_sample(output_len, output_len_std, output_len))
            head = f"Repeat lines of the text below in any order, for {n_out} tokens, without stopping:\n\n"
            left = n_in - len(self.tokenizer.encode(head))
            random.shuffle(order)
            parts = [head]
            pos = 0
            while left > 0:
                ids = self.line_ids[order[pos % len(order)]]
                pos += 1
                if len(ids) > left:
                    parts.append(self.tokenizer.decode(ids[:left]))
                else:
                    parts.append(self.lines[order[(pos - 1) % len(order)]])
                left -= len(ids)
            out.append(RequestRecord(chat_cmpl=_user("".join(parts), n_out, debug_config={"ignore_eos": True})))
        return out


class LoogleDataset(Dataset):
    """Long-document question answering: every document carries several questions, sent as one group so the
    later ones hit the prefix the first one cached. File: a list of ``{"input": document, "qa_pairs": [{"Q",
    "A"}, ...]}`` (``qa_pairs`` may be a string holding that list, as in the published dataset).
    Reference behaviour: ``LoogleDataset`` (``python/mlc_llm/bench/dataset.py:170-259``)."""

    require_fake_warmup = True
    TEMPLATES = {
        "shortdep_qa": "Answer the question from the text below.\n{input}\nQuestion: {Q}\nAnswer: ",
        "longdep_qa": "Answer the question from the text below.\n{input}\nQuestion: {Q}\nAnswer: ",
        "longdep_summarization": "Summarise the paper below.\n{input}\nSummary: ",
        "shortdep_cloze": "Fill in every '<mask-n>' of the question with an entity from the text below and answer "
                          "as a JSON object keyed by mask.\n{input}\nQuestion: {Q}\nAnswer: ",
    }

    def __init__(self, path: str, tokenizer, task: str = "shortdep_qa", truncate_length: int = 100000):
        import ast  # pylint: disable=import-outside-toplevel

        if task not in self.TEMPLATES:
            raise ValueError(f"unknown LooGLE task {task!r}; one of {sorted(self.TEMPLATES)}")
        self.tokenizer, self.template = tokenizer, self.TEMPLATES[task]
        self.docs = []
        for item in _records_of(path):
            qa = item.get("qa_pairs") or []
            if isinstance(qa, str):
                qa = ast.literal_eval(qa)
            if not qa:
                qa = [{"Q": "", "A": item.get("output", "") or ""}]
            ids = tokenizer.encode(item["input"])[:truncate_length]
            self.docs.append((item["input"], ids, [q.get("Q", "") for q in qa],
                              [max(1, len(tokenizer.encode(str(q.get("A", ""))))) for q in qa]))

    def generate_request_records(self, input_len, output_len, input_len_std=0.0, output_len_std=0.0):
        from .request_record import GroupedRequestRecord  # pylint: disable=import-outside-toplevel

        out = []
        for text, ids, questions, answer_lens in self.docs:
            if input_len is not None:
                want = _len_sample(input_len, input_len_std, len(ids))
                if len(ids) > want:
                    ids = ids[:want]
                    text = self.tokenizer.decode(ids)
            members = [RequestRecord(chat_cmpl=_user(self.template.format(input=text, Q=q),
                                                     _len_sample(output_len, output_len_std, alen)))
                       for q, alen in zip(questions, answer_lens)]
            out.append(GroupedRequestRecord(records=members))
        return out


class ReActDataset(Dataset):
    """Replay of recorded ReAct agent traces (not an agent): turn ``k`` of a trace sends the few-shot prefix,
    the question and the first ``k`` recorded steps, and asks for as many tokens as recorded step ``k`` has;
    the turns of one trace form a group, so each turn extends the prefix of the one before.
    File: a list of ``{"question": str, "steps": [str, ...]}``, optionally with one leading
    ``{"prefix": str}`` entry holding the few-shot examples (a short built-in instruction is used otherwise).
    Reference behaviour: ``ReActDataset`` (``python/mlc_llm/bench/dataset.py:405-581``)."""

    require_fake_warmup = True
    DEFAULT_PREFIX = ("Solve the question by alternating Thought, Action and Observation steps. An Action is one of "
                      "Search[entity], Lookup[keyword] or Finish[answer].\n")

    def __init__(self, path: str, tokenizer):
        self.tokenizer = tokenizer
        self.prefix = self.DEFAULT_PREFIX
        self.traces = []
        for item in _records_of(path):
            if "prefix" in item and "steps" not in item:
                self.prefix = item["prefix"]
                continue
            steps = [str(x) for x in item.get("steps", []) if str(x).strip()]
            if steps:
                self.traces.append((item.get("question", ""), steps,
                                    [max(1, len(tokenizer.encode(x))) for x in steps]))

    def generate_request_records(self, input_len, output_len, input_len_std=0.0, output_len_std=0.0):
        from .request_record import GroupedRequestRecord  # pylint: disable=import-outside-toplevel

        out = []
        for question, steps, lens in self.traces:
            members = []
            so_far = f"{self.prefix}Question: {question}\n"
            for step, n in zip(steps, lens):
                members.append(RequestRecord(chat_cmpl=_user(so_far, _len_sample(output_len, output_len_std, n),
                                                             debug_config={"ignore_eos": True})))
                so_far += step if step.endswith("\n") else step + "\n"
            out.append(GroupedRequestRecord(records=members))
        return out


class WildChatDataset(Dataset):
    """First user turn of every conversation with the length of the recorded assistant reply as the output
    length. File: a list of ``{"conversation": [{"role", "content"}, ...]}``.
    Reference behaviour: ``WildChatDataset`` (``python/mlc_llm/bench/dataset.py:584-702``)."""

    def __init__(self, path: str, tokenizer, apply_chat_template: bool = False):
        self.tokenizer = tokenizer
        self.items = []
        for item in _records_of(path):
            conv = item.get("conversation") or []
            if len(conv) < 2 or conv[0].get("role") != "user" or conv[1].get("role") != "assistant":
                continue
            prompt = conv[0]["content"]
            if apply_chat_template and hasattr(tokenizer, "apply_chat_template"):
                prompt = tokenizer.apply_chat_template([{"role": "user", "content": prompt}],
                                                       add_generation_prompt=True, tokenize=False)
            p_ids, c_len = tokenizer.encode(prompt), len(tokenizer.encode(conv[1]["content"]))
            if len(p_ids) >= 4 and c_len >= 4:
                self.items.append((prompt, p_ids, c_len))
        random.shuffle(self.items)

    def generate_request_records(self, input_len, output_len, input_len_std=0.0, output_len_std=0.0):
        out = []
        for prompt, ids, c_len in self.items:
            if input_len is not None:
                want = _len_sample(input_len, input_len_std, len(ids))
                if len(ids) < want:
                    continue
                prompt = self.tokenizer.decode(ids[:want])
            out.append(RequestRecord(chat_cmpl=_user(prompt, _len_sample(output_len, output_len_std, c_len))))
        return out


class AzureLLMInferenceDataset(Dataset):
    """Replay of an Azure LLM inference trace: a CSV with ``TIMESTAMP``, ``ContextTokens`` and
    ``GeneratedTokens`` columns. Only arrival times and lengths are recorded, so prompts are random token ids
    adjusted until decode + encode gives the recorded length; each request keeps its offset from the first
    arrival as its send time. Reference behaviour: ``AzureLLMInferenceDataset``
    (``python/mlc_llm/bench/dataset.py:705-797``)."""

    timestamp_available = True

    def __init__(self, path: str, tokenizer, truncate_length: int = 100000):
        import csv  # pylint: disable=import-outside-toplevel
        from datetime import datetime  # pylint: disable=import-outside-toplevel

        self.tokenizer = tokenizer
        self.rows = []
        with open(path, newline="", encoding="utf-8") as f:
            for row in csv.DictReader(f):
                n_in, n_out = int(float(row["ContextTokens"])), int(float(row["GeneratedTokens"]))
                if n_in < 4 or n_out < 4:
                    continue
                stamp = row["TIMESTAMP"].strip().rstrip("Z")
                if "." in stamp:
                    whole, frac = stamp.split(".", 1)
                    stamp = whole + "." + frac[:6]   # the trace has 7 fractional digits
                    when = datetime.strptime(stamp, "%Y-%m-%d %H:%M:%S.%f")
                else:
                    when = datetime.strptime(stamp, "%Y-%m-%d %H:%M:%S")
                self.rows.append((when, min(n_in, truncate_length), min(n_out, truncate_length)))
        self.rows.sort(key=lambda r: r[0])

    def _prompt_of_length(self, n: int, vocab: int) -> str:
        ids = np.random.randint(0, vocab, size=n).tolist()
        for _ in range(16):
            text = self.tokenizer.decode(ids)
            back = self.tokenizer.encode(text)
            if len(back) == n:
                return text
            ids = back[:n] if len(back) > n else back + np.random.randint(0, vocab, size=n - len(back)).tolist()
        return self.tokenizer.decode(ids)

    def generate_request_records(self, input_len, output_len, input_len_std=0.0, output_len_std=0.0):
        if not self.rows:
            return []
        vocab = getattr(self.tokenizer, "vocab_size", 32000)
        vocab = int(vocab() if callable(vocab) else vocab)
        t0 = self.rows[0][0]
        out = []
        for when, n_in, n_out in self.rows:
            if input_len is not None:
                if n_in < input_len + 4 * input_len_std:
                    continue
                n_in = max(1, _len_sample(input_len, input_len_std, n_in))
            if output_len is not None:
                n_out = max(1, _len_sample(output_len, output_len_std, n_out))
            out.append(RequestRecord(chat_cmpl=_user(self._prompt_of_length(n_in, vocab), n_out),
                                     timestamp=(when - t0).total_seconds()))
        return out


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
    if name == "llmperf":
        return LLMPerfDataset(args.dataset_path, (args.num_requests + args.num_warmup_requests) * 4, tokenizer)
    if name == "loogle":
        return LoogleDataset(args.dataset_path, tokenizer, getattr(args, "loogle_task", None) or "shortdep_qa")
    if name == "react":
        return ReActDataset(args.dataset_path, tokenizer)
    if name == "wildchat":
        return WildChatDataset(args.dataset_path, tokenizer, args.apply_chat_template)
    if name == "azure-llm-inference":
        return AzureLLMInferenceDataset(args.dataset_path, tokenizer)
    raise ValueError(f"unknown dataset {name!r}; one of {SUPPORTED_DATASET}")
