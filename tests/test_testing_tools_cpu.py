"""Debugging tools: operator dump per step (DebugChat) and operator-by-operator device comparison."""
import glob
import os

import numpy as np

from mlc_llm_b200.testing.debug_chat import DebugChat, DebugInstrument
from mlc_llm_b200.testing.debug_compare import compare

MODEL = "random://tiny-llama?quant=q0f32&seed=3"


def test_debug_chat_dumps_every_operator_call(tmp_path):
    chat = DebugChat(MODEL, str(tmp_path), "cpu")
    ids = chat.generate(list(range(100, 112)), 3)
    assert len(ids) == 3
    assert sorted(os.listdir(tmp_path)) == ["decode_0", "decode_1", "prefill"]
    files = sorted(glob.glob(str(tmp_path / "prefill" / "*.npz")))
    names = [os.path.basename(f) for f in files]
    assert any("_linear" in n for n in names) and any("_paged_attention" in n for n in names)
    first_linear = np.load([f for f in files if "_linear" in f][0])
    assert first_linear["arg_0"].shape == (12, 256) and "out_0" in first_linear.files
    assert not chat.instrument.first_nan_occurred


def test_debug_instrument_flags_nan(tmp_path):
    import torch

    inst = DebugInstrument(str(tmp_path))
    inst("fake_op", (torch.ones(2),), {}, torch.tensor([1.0, float("nan")]))
    assert inst.first_nan_occurred and "NaN" in inst.log[0]


def test_debug_compare_reports_per_operator_deviation():
    cmp = compare(MODEL, list(range(50, 60)), "cpu", "cpu", generate_len=2)
    s = cmp.summary()
    assert s["linear"]["calls"] >= 9 and s["linear"]["mismatches"] == 0 and s["linear"]["max_abs_err"] == 0.0
    assert "rmsnorm" in s or "add_rmsnorm" in s
