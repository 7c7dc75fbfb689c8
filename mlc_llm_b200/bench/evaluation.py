"""Accuracy checks through the engine's chat API: GSM8K (grade-school arithmetic, free-form answer) and
MMLU (four-way multiple choice), read from local dataset files.

Reference: ``python/mlc_llm/bench/evaluation/gsm8k.py`` and ``mmlu.py`` (few-shot prompts sent through
``AsyncMLCEngine`` with bounded concurrency, answers extracted with regular expressions, a JSON summary
written next to the per-question log).

    python -m mlc_llm_b200.bench.evaluation gsm8k --model <dir> --dataset test.jsonl --n-shot 4
    python -m mlc_llm_b200.bench.evaluation mmlu  --model <dir> --dataset <dir with *_test.csv> --subjects all

GSM8K files are JSON lines with ``question`` and ``answer`` (the answer ends in ``#### <number>``); MMLU
files are CSV rows ``question, A, B, C, D, answer letter``.
"""

from __future__ import annotations

import argparse
import asyncio
import csv
import glob
import json
import os
import re
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

INVALID = "[invalid]"
_NUMBER = re.compile(r"-?\$?\d[\d,]*(?:\.\d+)?")
_TRUTH = re.compile(r"####\s*(-?[\d.,]+)")
_STATED = re.compile(r"[Tt]he answer is\s*\$?(-?[\d.,]+)")
_CHOICE = re.compile(r"\b([ABCD])\b")


def _clean_number(text: str) -> str:
    text = text.strip().lstrip("$").replace(",", "").rstrip(".")
    if "." in text:
        text = text.rstrip("0").rstrip(".")
    return text or INVALID


def gsm8k_truth(answer: str) -> str:
    """The number after ``####`` in a GSM8K reference solution."""
    m = _TRUTH.search(answer)
    return _clean_number(m.group(1)) if m else INVALID


def gsm8k_answer(text: str, strict: bool = False) -> str:
    """The model's number: the one after "The answer is" (``strict``), else the last number in the text."""
    m = _STATED.search(text)
    if m:
        return _clean_number(m.group(1))
    if strict:
        return INVALID
    found = _NUMBER.findall(text)
    return _clean_number(found[-1]) if found else INVALID


def mmlu_answer(text: str) -> str:
    """The first stand-alone letter A-D of the reply."""
    m = _CHOICE.search(text.strip())
    return m.group(1) if m else INVALID


def gsm8k_prompt(question: str, shots: Sequence[Dict[str, str]]) -> str:
    parts = []
    for s in shots:
        worked = s["answer"].split("####")[0].strip()
        parts.append(f"Q: {s['question']}\nA: {worked} The answer is {gsm8k_truth(s['answer'])}.\n")
    parts.append(f"Q: {question}\nA:")
    return "\n".join(parts)


def mmlu_prompt(subject: str, row: Sequence[str], shots: Sequence[Sequence[str]]) -> str:
    def block(r: Sequence[str], with_answer: bool) -> str:
        text = f"{r[0]}\nA. {r[1]}\nB. {r[2]}\nC. {r[3]}\nD. {r[4]}\nAnswer:"
        return text + (f" {r[5]}\n" if with_answer else "")

    head = f"The following are multiple choice questions (with answers) about {subject.replace('_', ' ')}.\n"
    return head + "\n".join(block(s, True) for s in shots) + ("\n" if shots else "") + block(row, False)


def load_gsm8k(path: str) -> List[Dict[str, str]]:
    with open(path, encoding="utf-8") as f:
        return [json.loads(line) for line in f if line.strip()]


def load_mmlu(directory: str, subjects: Optional[Sequence[str]] = None) -> Dict[str, List[List[str]]]:
    """``{subject: rows}`` from ``<subject>_test.csv`` (or ``<subject>.csv``) files of a directory."""
    out: Dict[str, List[List[str]]] = {}
    for path in sorted(glob.glob(os.path.join(directory, "*.csv"))):
        name = os.path.basename(path)[: -len(".csv")]
        subject = name[: -len("_test")] if name.endswith("_test") else name
        if subjects and "all" not in subjects and subject not in subjects:
            continue
        with open(path, encoding="utf-8", newline="") as f:
            out[subject] = [r for r in csv.reader(f) if len(r) >= 6]
    return out


async def _ask_all(engine, prompts: Sequence[str], max_tokens: int, concurrency: int,
                   stop: Optional[List[str]] = None) -> List[str]:
    """Send every prompt as a one-turn chat, at most ``concurrency`` in flight; replies in prompt order."""
    gate = asyncio.Semaphore(max(1, concurrency))
    replies: List[str] = [""] * len(prompts)

    async def one(i: int, prompt: str) -> None:
        async with gate:
            resp = await engine.chat.completions.create(messages=[{"role": "user", "content": prompt}],
                                                        max_tokens=max_tokens, temperature=0.0, stop=stop)
            replies[i] = resp.choices[0].message.content or ""

    await asyncio.gather(*(one(i, p) for i, p in enumerate(prompts)))
    return replies


def evaluate_gsm8k(engine, rows: Sequence[Dict[str, str]], n_shot: int = 4, max_tokens: int = 256,
                   concurrency: int = 16, strict: bool = False, ask: Optional[Callable] = None) -> Dict[str, Any]:
    """Accuracy on GSM8K rows; the first ``n_shot`` rows become worked examples and are not scored.
    ``ask(prompts) -> replies`` replaces the engine call (used by tests and by REST-endpoint runs)."""
    shots, scored = list(rows[:n_shot]), list(rows[n_shot:])
    prompts = [gsm8k_prompt(r["question"], shots) for r in scored]
    replies = ask(prompts) if ask is not None else asyncio.run(
        _ask_all(engine, prompts, max_tokens, concurrency, stop=["Q:", "\n\n\n"]))
    log, correct, invalid = [], 0, 0
    for r, reply in zip(scored, replies):
        want, got = gsm8k_truth(r["answer"]), gsm8k_answer(reply, strict)
        ok = got != INVALID and got == want
        correct += ok
        invalid += got == INVALID
        log.append({"question": r["question"], "reply": reply, "extracted": got, "truth": want, "correct": bool(ok)})
    n = max(1, len(scored))
    return {"task": "gsm8k", "num_questions": len(scored), "n_shot": n_shot, "accuracy": correct / n,
            "invalid_rate": invalid / n, "log": log}


def evaluate_mmlu(engine, subjects: Dict[str, List[List[str]]], n_shot: int = 5, concurrency: int = 16,
                  ask: Optional[Callable] = None) -> Dict[str, Any]:
    """Per-subject and overall accuracy; the first ``n_shot`` rows of a subject are its examples."""
    index: List[Tuple[str, List[str]]] = []
    prompts: List[str] = []
    for subject, rows in subjects.items():
        shots = rows[:n_shot]
        for row in rows[n_shot:]:
            index.append((subject, row))
            prompts.append(mmlu_prompt(subject, row, shots))
    replies = ask(prompts) if ask is not None else asyncio.run(_ask_all(engine, prompts, 4, concurrency))
    per: Dict[str, List[int]] = {}
    for (subject, row), reply in zip(index, replies):
        hit = mmlu_answer(reply) == row[5].strip().upper()
        tally = per.setdefault(subject, [0, 0])
        tally[0] += hit
        tally[1] += 1
    total = sum(t[1] for t in per.values())
    return {"task": "mmlu", "num_questions": total, "n_shot": n_shot,
            "accuracy": sum(t[0] for t in per.values()) / max(1, total),
            "per_subject": {s: t[0] / max(1, t[1]) for s, t in per.items()}}


def main(argv: Optional[Sequence[str]] = None) -> Dict[str, Any]:
    parser = argparse.ArgumentParser("mlc_llm_b200.bench.evaluation")
    parser.add_argument("task", choices=["gsm8k", "mmlu"])
    parser.add_argument("--model", required=True)
    parser.add_argument("--model-lib", default=None)
    parser.add_argument("--device", default="auto")
    parser.add_argument("--dataset", required=True, help="GSM8K .jsonl file, or a directory of MMLU .csv files")
    parser.add_argument("--subjects", nargs="*", default=["all"])
    parser.add_argument("--n-shot", type=int, default=None)
    parser.add_argument("--max-tokens", type=int, default=256)
    parser.add_argument("--concurrency", type=int, default=16)
    parser.add_argument("--strict", action="store_true", help='GSM8K: only accept "The answer is <n>"')
    parser.add_argument("--limit", type=int, default=0, help="score at most this many questions")
    parser.add_argument("--output", default=None, help="write the summary (and the GSM8K log) to this JSON file")
    args = parser.parse_args(argv)
    from ..serve.engine import AsyncMLCEngine  # pylint: disable=import-outside-toplevel

    engine = AsyncMLCEngine(args.model, args.device, model_lib=args.model_lib, mode="server")
    try:
        if args.task == "gsm8k":
            rows = load_gsm8k(args.dataset)
            shot = 4 if args.n_shot is None else args.n_shot
            if args.limit:
                rows = rows[: shot + args.limit]
            result = evaluate_gsm8k(engine, rows, shot, args.max_tokens, args.concurrency, args.strict)
        else:
            subjects = load_mmlu(args.dataset, args.subjects)
            shot = 5 if args.n_shot is None else args.n_shot
            if args.limit:
                subjects = {s: r[: shot + args.limit] for s, r in subjects.items()}
            result = evaluate_mmlu(engine, subjects, shot, args.concurrency)
    finally:
        engine.terminate()
    if args.output:
        with open(args.output, "w", encoding="utf-8") as f:
            json.dump(result, f, indent=2)
    print(json.dumps({k: v for k, v in result.items() if k != "log"}))
    return result


if __name__ == "__main__":
    main()
