"""``mlc_llm_b200 calibrate``: activation ranges per linear layer, stored in a tensor cache."""
import json
import os

import torch

from mlc_llm_b200 import ops
from mlc_llm_b200.cli import calibrate as calibrate_cli
from mlc_llm_b200.interface.calibrate import CalibrationObserver, FP8_E4M3_MAX
from mlc_llm_b200.loader.tensor_cache import TensorCache, dump_tensor_cache, update_tensor_cache


def test_observer_keeps_running_max_per_layer():
    class _Model:
        class p:  # pylint: disable=invalid-name
            linears = {"a": ops.dense_weight(torch.eye(4)), "b": ops.dense_weight(torch.eye(4))}

    obs = CalibrationObserver()
    obs.watch(_Model)
    ops.set_linear_observer(obs)
    try:
        ops.linear(torch.tensor([[1.0, -3.0, 0.5, 0.0]]), _Model.p.linears["a"])
        ops.linear(torch.tensor([[2.0, 1.0, 0.5, 0.0]]), _Model.p.linears["a"])
        ops.linear(torch.tensor([[0.25, 0.0, 0.0, 0.0]]), _Model.p.linears["b"])
    finally:
        ops.set_linear_observer(None)
    scales = dict(obs.scales())
    assert torch.allclose(scales["a.q_calibration_scale"], torch.tensor([3.0 / FP8_E4M3_MAX]))
    assert torch.allclose(scales["b.q_calibration_scale"], torch.tensor([0.25 / FP8_E4M3_MAX]))


def test_update_tensor_cache_adds_and_replaces(tmp_path):
    out = str(tmp_path / "cache")
    dump_tensor_cache(iter([("w", torch.arange(6, dtype=torch.float16).reshape(2, 3)),
                            ("s", torch.ones(2, dtype=torch.float32))]), out, encode_format="raw")
    update_tensor_cache(iter([("s", torch.full((2,), 5.0)), ("extra", torch.tensor([7.0]))]), out,
                        encode_format="raw")
    tc = TensorCache(out)
    assert sorted(tc.names()) == ["extra", "s", "w"]
    assert tc.get("s").tolist() == [5.0, 5.0] and tc.get("extra").tolist() == [7.0]
    assert tc.get("w").tolist() == [[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]]


def test_calibrate_command_on_tiny_model(tmp_path, monkeypatch):
    monkeypatch.delenv("MLCB_CUDA_GRAPH", raising=False)
    data = [{"conversations": [{"value": f"tell me about item {i} please now"},
                               {"value": f"it is a thing with number {i} ok"}]} for i in range(6)]
    data.append({"conversations": [{"value": "only one turn"}]})
    ds = tmp_path / "ds.json"
    ds.write_text(json.dumps(data))
    out = str(tmp_path / "calib")
    calibrate_cli.main(["random://tiny-llama?quant=q0f32&seed=5", "--device", "cpu", "-o", out,
                        "--dataset", str(ds), "--num-calibration-samples", "3",
                        "--overrides", "max_num_sequence=4;max_total_seq_length=1024;prefill_chunk_size=64"])
    tc = TensorCache(out)
    names = tc.names()
    assert "lm_head.q_calibration_scale" in names
    assert "model.layers.0.self_attn.qkv_proj.q_calibration_scale" in names
    assert all(float(tc.get(n)) > 0 for n in names)
    assert "MLCB_CUDA_GRAPH" not in os.environ  # the temporary switches were put back
