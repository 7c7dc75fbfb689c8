"""Workload sources of the load generator: each dataset kind of the reference, read from a small local file,
and the executors' handling of grouped (multi-turn / shared-document) records."""
import asyncio
import json
import random

import numpy as np

from mlc_llm_b200.bench import dataset as D
from mlc_llm_b200.bench.request_processor import (AttachModelName, AttachSamplingOptions,
                                                  FixedConcurrentRequestExecutor, SampleRequests)
from mlc_llm_b200.bench.request_record import GroupedRequestRecord, Metrics, RequestRecord


class WordTokenizer:
    """One token per whitespace-separated word (ids are stable hashes into a small vocabulary)."""

    vocab_size = 5000

    def __init__(self):
        self.words = {}

    def encode(self, text):
        out = []
        for w in text.split():
            out.append(self.words.setdefault(w, len(self.words) % self.vocab_size))
        return out

    def decode(self, ids):
        back = {v: k for k, v in self.words.items()}
        return " ".join(back.get(i, f"w{i}") for i in ids)


def _n_tokens(tok, record):
    return len(tok.encode(record.chat_cmpl["messages"][0]["content"]))


def test_llmperf_prompts_have_the_requested_length(tmp_path):
    random.seed(0)
    np.random.seed(0)
    path = tmp_path / "sonnet.txt"
    path.write_text("\n".join(f"line {i} of some verse with seven words" for i in range(50)) + "\n")
    tok = WordTokenizer()
    ds = D.LLMPerfDataset(str(path), 6, tok)
    recs = ds.generate_request_records(200, 64, 0.0, 0.0)
    assert len(recs) == 6
    for r in recs:
        assert _n_tokens(tok, r) == 200
        assert r.chat_cmpl["max_tokens"] == 64 and r.chat_cmpl["debug_config"]["ignore_eos"]
    assert len({r.chat_cmpl["messages"][0]["content"] for r in recs}) > 1   # shuffled per request


def test_loogle_groups_the_questions_of_a_document(tmp_path):
    path = tmp_path / "loogle.jsonl"
    docs = [{"input": " ".join(f"d{k}w{i}" for i in range(300)),
             "qa_pairs": str([{"Q": f"question {j}", "A": "an answer of five words"} for j in range(3)])}
            for k in range(2)]
    path.write_text("\n".join(json.dumps(d) for d in docs))
    tok = WordTokenizer()
    recs = D.LoogleDataset(str(path), tok).generate_request_records(100, None)
    assert len(recs) == 2 and all(isinstance(g, GroupedRequestRecord) and len(g.records) == 3 for g in recs)
    a, b = recs[0].records[0].chat_cmpl, recs[0].records[1].chat_cmpl
    assert a["max_tokens"] == 5
    # the members share the (truncated) document and differ in the question
    shared = a["messages"][0]["content"].split("Question:")[0]
    assert shared == b["messages"][0]["content"].split("Question:")[0] and "d0w99" in shared and "d0w100" not in shared
    assert a["messages"][0]["content"] != b["messages"][0]["content"]


def test_react_turns_extend_one_another(tmp_path):
    path = tmp_path / "react.json"
    path.write_text(json.dumps([{"prefix": "FEWSHOT "},
                                {"question": "who?", "steps": ["Thought 1: a b c", "Action 1: Search[x]",
                                                               "Observation 1: found it here"]}]))
    tok = WordTokenizer()
    (group,) = D.ReActDataset(str(path), tok).generate_request_records(None, None)
    texts = [m.chat_cmpl["messages"][0]["content"] for m in group.records]
    assert texts[0].startswith("FEWSHOT Question: who?") and len(texts) == 3
    assert texts[1].startswith(texts[0]) and texts[2].startswith(texts[1]) and "Search[x]" in texts[2]
    assert [m.chat_cmpl["max_tokens"] for m in group.records] == [5, 3, 5]


def test_wildchat_and_azure_trace(tmp_path):
    tok = WordTokenizer()
    wc = tmp_path / "wildchat.jsonl"
    rows = [{"conversation": [{"role": "user", "content": "tell me a story about four things"},
                              {"role": "assistant", "content": "once upon a time there was"}]},
            {"conversation": [{"role": "user", "content": "hi"}]},
            {"conversation": [{"role": "assistant", "content": "x"}, {"role": "user", "content": "y"}]}]
    wc.write_text("\n".join(json.dumps(r) for r in rows))
    recs = D.WildChatDataset(str(wc), tok).generate_request_records(None, None)
    assert len(recs) == 1 and recs[0].chat_cmpl["max_tokens"] == 6
    az = tmp_path / "trace.csv"
    az.write_text("TIMESTAMP,ContextTokens,GeneratedTokens\n"
                  "2023-11-16 18:15:46.6805900,40,12\n2023-11-16 18:15:47.1805900,3,50\n"
                  "2023-11-16 18:15:49.6805900,25,8\n")
    ds = D.AzureLLMInferenceDataset(str(az), tok)
    recs = ds.generate_request_records(None, None)
    assert ds.timestamp_available and [r.timestamp for r in recs] == [0.0, 3.0]
    assert [r.chat_cmpl["max_tokens"] for r in recs] == [12, 8]
    assert [_n_tokens(tok, r) for r in recs] == [40, 25]


def test_groups_are_sent_in_order_and_flattened():
    order = []

    class FakeEndpoint:
        async def __aenter__(self):
            return self

        async def __aexit__(self, *exc):
            return False

        async def __call__(self, rec):
            await asyncio.sleep(0.001)
            order.append(rec.chat_cmpl["messages"][0]["content"])
            rec.metrics = Metrics(success=True)
            return rec

    def group(tag, n):
        return GroupedRequestRecord(records=[RequestRecord(chat_cmpl=D._user(f"{tag}{i}", 4)) for i in range(n)])

    records = [group("a", 3), RequestRecord(chat_cmpl=D._user("solo", 4)), group("b", 2)]
    records = AttachSamplingOptions(0.0, 1.0, True)(AttachModelName("m")(records))
    done = FixedConcurrentRequestExecutor(FakeEndpoint, 2)(records)
    assert len(done) == 6 and all(r.chat_cmpl["model"] == "m" and r.chat_cmpl["debug_config"]["ignore_eos"]
                                  for r in done)
    assert [x for x in order if x.startswith("a")] == ["a0", "a1", "a2"]
    assert [x for x in order if x.startswith("b")] == ["b0", "b1"]
    # a short dataset is recycled without sharing objects between the copies
    more = SampleRequests(5)([group("c", 2)])
    assert len(more) == 5 and more[0].records[0] is not more[1].records[0]
