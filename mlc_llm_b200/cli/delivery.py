"""Continuous model delivery: run ``gen_config`` + ``convert_weight`` for every (model, quantisation)
pair of a spec file that the delivery log does not list yet (reference: ``python/mlc_llm/cli/delivery.py``,
same spec and log formats).

    python -m mlc_llm_b200.cli.delivery --spec model-delivery-config.json --log model-delivered-log.json \\
        --output <dir> [--username <hf-user> --token <hf-token>] [--dry-run]

``model`` entries are local HuggingFace checkpoint directories or ``HF://org/name`` references.  A hub
reference is resolved through the download cache (``support/download_cache.py``); uploading the result needs
``huggingface_hub`` and credentials, otherwise the converted models stay under ``--output`` and the log
records them as delivered locally.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Any, Dict, List, Optional, Union

from pydantic import BaseModel, Field

GEN_CONFIG_OPTIONAL_ARGS = ["context_window_size", "sliding_window_size", "prefill_chunk_size",
                            "attention_sink_size", "tensor_parallel_shards", "pipeline_parallel_stages"]


class OverrideConfigs(BaseModel):
    context_window_size: Optional[int] = None
    sliding_window_size: Optional[int] = None
    prefill_chunk_size: Optional[int] = None
    attention_sink_size: Optional[int] = None
    tensor_parallel_shards: Optional[int] = None
    pipeline_parallel_stages: Optional[int] = None


class ModelDeliveryTask(BaseModel):
    """``{"model_id": "...", "model": "HF://org/name" | "<dir>", "conv_template": "...",
    "quantization": ["q4f16_1"], "overrides": {"q4f16_1": {"context_window_size": 512}}}``"""

    model_id: str
    model: str
    conv_template: str
    quantization: Union[List[str], str] = Field(default_factory=list)
    overrides: Dict[str, OverrideConfigs] = Field(default_factory=dict)
    destination: Optional[str] = None
    gen_config_only: Optional[bool] = False


class ModelDeliveryList(BaseModel):
    tasks: List[ModelDeliveryTask]
    default_destination: Optional[str] = None
    default_quantization: List[str] = Field(default_factory=list)
    default_overrides: Dict[str, OverrideConfigs] = Field(default_factory=dict)

    @classmethod
    def from_json(cls, d: Dict[str, Any]) -> "ModelDeliveryList":
        return cls.model_validate(d)

    def to_json(self) -> Dict[str, Any]:
        return self.model_dump(exclude_none=True)


def get_current_log(log: str) -> ModelDeliveryList:
    if not os.path.exists(log):
        current = ModelDeliveryList(tasks=[])
        with open(log, "w", encoding="utf-8") as f:
            json.dump(current.to_json(), f, indent=4)
        return current
    with open(log, encoding="utf-8") as f:
        return ModelDeliveryList.from_json(json.load(f))


def generate_model_delivery_diff(spec: ModelDeliveryList, log: ModelDeliveryList) -> ModelDeliveryList:
    """Tasks of ``spec`` not yet in ``log``, one per quantisation.  A pair already delivered with the same
    overrides but another conversation template only needs its config regenerated."""
    diff: List[ModelDeliveryTask] = []
    for task in spec.tasks:
        overrides = {**spec.default_overrides, **task.overrides}
        quant = [task.quantization] if isinstance(task.quantization, str) else list(task.quantization)
        delivered, config_only = set(), set()
        for done in (t for t in log.tasks if t.model_id == task.model_id):
            q = done.quantization if isinstance(done.quantization, str) else (done.quantization or [None])[0]
            if done.overrides.get(q, OverrideConfigs()) == overrides.get(q, OverrideConfigs()):
                (delivered if done.conv_template == task.conv_template else config_only).add(q)
        for q in sorted((set(spec.default_quantization) | set(quant)) - delivered):
            t = task.model_copy()
            t.quantization = [q]
            t.overrides = {q: overrides.get(q, OverrideConfigs())}
            t.gen_config_only = bool(t.gen_config_only) or q in config_only
            diff.append(t)
    out = spec.model_copy()
    out.default_quantization, out.default_overrides, out.tasks = [], {}, diff
    return out


def _resolve_source(model: str, hf_local_dir: Optional[str]) -> str:
    if model.startswith("HF://"):
        from ..support.download_cache import get_or_download_model  # pylint: disable=import-outside-toplevel

        return str(get_or_download_model(model))
    if os.path.isdir(model):
        return model
    if hf_local_dir and os.path.isdir(os.path.join(hf_local_dir, model)):
        return os.path.join(hf_local_dir, model)
    raise FileNotFoundError(f"model source {model!r} is neither a directory nor an HF:// reference")


def run_task(task: ModelDeliveryTask, output: str, hf_local_dir: Optional[str] = None) -> str:
    """gen_config (+ convert_weight) of one (model, quantisation) pair; returns the model directory."""
    from ..interface.convert_weight import convert_weight  # pylint: disable=import-outside-toplevel
    from ..interface.gen_config import gen_config  # pylint: disable=import-outside-toplevel

    q = task.quantization[0] if isinstance(task.quantization, list) else task.quantization
    src = _resolve_source(task.model, hf_local_dir)
    out_dir = os.path.join(output, f"{task.model_id}-{q}-MLC")
    os.makedirs(out_dir, exist_ok=True)
    ov = task.overrides.get(q, OverrideConfigs())
    kwargs = {k: getattr(ov, k) for k in GEN_CONFIG_OPTIONAL_ARGS}
    gen_config(src, "auto", q, task.conv_template, disaggregation=None, max_batch_size=128, output=out_dir,
               **kwargs)
    if not task.gen_config_only:
        convert_weight(src, q, output=out_dir, verbose=False)
    return out_dir


def _upload(api, username: str, task: ModelDeliveryTask, model_dir: str) -> str:
    q = task.quantization[0]
    repo = task.destination or f"{username}/{task.model_id}-{q}-MLC"
    api.create_repo(repo_id=repo, private=False, exist_ok=True)
    api.upload_folder(folder_path=model_dir, repo_id=repo, ignore_patterns=["logs.txt"])
    return repo


def deliver(spec: ModelDeliveryList, log: str, output: str, username: Optional[str] = None, api=None,
            hf_local_dir: Optional[str] = None, dry_run: bool = False) -> List[str]:
    """Process the spec; returns the model directories produced."""
    diff = generate_model_delivery_diff(spec, get_current_log(log))
    if dry_run:
        print(json.dumps(diff.to_json(), indent=2))
        return []
    produced, failed = [], []
    delivered = get_current_log(log)
    for i, task in enumerate(diff.tasks, 1):
        print(f"[{i}/{len(diff.tasks)}] {task.model_id} {task.quantization[0]}")
        try:
            model_dir = run_task(task, output, hf_local_dir)
            if api is not None and username:
                task.destination = _upload(api, username, task, model_dir)
                shutil.rmtree(model_dir, ignore_errors=True)
            else:
                task.destination = model_dir
            produced.append(model_dir)
        except Exception as err:  # pylint: disable=broad-except
            failed.append((task.model_id, task.quantization[0], str(err)))
            continue
        entry = task.model_copy()
        entry.quantization = task.quantization[0]
        delivered.tasks.append(entry)
        with open(log, "w", encoding="utf-8") as f:
            json.dump(delivered.to_json(), f, indent=4)
    for model_id, q, why in failed:
        print(f"FAILED {model_id} {q}: {why}")
    return produced


def main(argv=None) -> None:
    p = argparse.ArgumentParser("mlc_llm_b200 continuous model delivery")
    p.add_argument("--username", type=str, default=None, help="HuggingFace user or organisation to upload to")
    p.add_argument("--token", type=str, default=os.environ.get("HF_TOKEN"))
    p.add_argument("--spec", type=str, default="model-delivery-config.json")
    p.add_argument("--log", type=str, default="model-delivered-log.json")
    p.add_argument("--output", type=str, required=True)
    p.add_argument("--hf-local-dir", type=str, default=None)
    p.add_argument("--dry-run", action="store_true")
    a = p.parse_args(argv)
    with open(a.spec, encoding="utf-8") as f:
        spec = ModelDeliveryList.from_json(json.load(f))
    api = None
    if a.username and a.token and not a.dry_run:
        try:
            from huggingface_hub import HfApi  # pylint: disable=import-outside-toplevel

            api = HfApi(token=a.token)
        except ImportError:
            print("huggingface_hub is not installed: models stay under --output")
    deliver(spec, a.log, a.output, a.username, api, a.hf_local_dir, a.dry_run)


if __name__ == "__main__":
    main()
