"""Accuracy-evaluation helpers: answer extraction, few-shot prompts, scoring, and one run through an engine."""
import csv
import json

from mlc_llm_b200.bench import evaluation as ev


def test_answer_extraction():
    assert ev.gsm8k_truth("She has 3 + 4 = 7 apples.\n#### 7") == "7"
    assert ev.gsm8k_truth("...\n#### 1,250.00") == "1250"
    assert ev.gsm8k_answer("So 3 + 4 = 7. The answer is 7.") == "7"
    assert ev.gsm8k_answer("They earn $1,250 in total") == "1250"
    assert ev.gsm8k_answer("no idea") == ev.INVALID
    assert ev.gsm8k_answer("maybe 12", strict=True) == ev.INVALID
    assert ev.mmlu_answer(" B. because") == "B" and ev.mmlu_answer("The answer is (C)") == "C"
    assert ev.mmlu_answer("unsure") == ev.INVALID


def test_scoring_with_a_scripted_model(tmp_path):
    rows = [{"question": f"What is {i} + {i}?", "answer": f"{i} + {i} = {2 * i}\n#### {2 * i}"} for i in range(1, 7)]
    path = tmp_path / "gsm.jsonl"
    path.write_text("\n".join(json.dumps(r) for r in rows))
    loaded = ev.load_gsm8k(str(path))
    seen = []

    def ask(prompts):
        seen.extend(prompts)
        # right on the first two scored questions, wrong on the third, no number on the fourth
        return ["The answer is 6.", "so it is 8", "The answer is 11.", "I do not know"]

    res = ev.evaluate_gsm8k(None, loaded, n_shot=2, ask=ask)
    assert res["num_questions"] == 4 and res["accuracy"] == 0.5 and res["invalid_rate"] == 0.25
    assert seen[0].count("Q:") == 3 and "The answer is 2." in seen[0] and seen[0].endswith("Q: What is 3 + 3?\nA:")

    mm = tmp_path / "mmlu"
    mm.mkdir()
    with open(mm / "toy_math_test.csv", "w", newline="") as f:
        w = csv.writer(f)
        for i in range(4):
            w.writerow([f"{i} + 1 = ?", str(i + 1), str(i + 2), str(i + 3), str(i + 4), "A"])
    subjects = ev.load_mmlu(str(mm))
    assert list(subjects) == ["toy_math"]
    res = ev.evaluate_mmlu(None, subjects, n_shot=1, ask=lambda prompts: ["A", " B", "A."])
    assert res["num_questions"] == 3 and abs(res["accuracy"] - 2 / 3) < 1e-9
    assert abs(res["per_subject"]["toy_math"] - 2 / 3) < 1e-9


def test_gsm8k_through_an_engine(tmp_path):
    rows = [{"question": f"What is {i} + 1?", "answer": f"#### {i + 1}"} for i in range(4)]
    path = tmp_path / "gsm.jsonl"
    path.write_text("\n".join(json.dumps(r) for r in rows))
    out = tmp_path / "res.json"
    res = ev.main(["gsm8k", "--model", "random://tiny-llama?quant=q0f32&seed=1", "--device", "cpu",
                   "--dataset", str(path), "--n-shot", "1", "--max-tokens", "6", "--concurrency", "2",
                   "--output", str(out)])
    assert res["num_questions"] == 3 and 0.0 <= res["accuracy"] <= 1.0 and len(res["log"]) == 3
    assert json.load(open(out))["task"] == "gsm8k"
