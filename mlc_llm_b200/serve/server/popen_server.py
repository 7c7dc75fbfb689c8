"""Run ``python -m mlc_llm_b200 serve`` as a child process and wait until it answers (reference:
``python/mlc_llm/serve/server/popen_server.py:16-200``).  Used by the router, the load generator and
the REST tests."""

from __future__ import annotations

import dataclasses
import os
import subprocess
import sys
import time
from typing import Dict, List, Optional

import requests


_OVERRIDE_KEYS = {"max_num_sequence", "max_total_sequence_length", "max_single_sequence_length",
                  "prefill_chunk_size", "sliding_window_size", "attention_sink_size", "max_history_size",
                  "gpu_memory_utilization", "spec_draft_length", "spec_tree_width",
                  "prefix_cache_max_num_recycling_seqs", "tensor_parallel_shards", "pipeline_parallel_stages", "opt"}


class PopenServer:  # pylint: disable=too-many-instance-attributes
    def __init__(self, model: str, device: str = "auto", *, model_lib: Optional[str] = None,
                 mode: str = "local", engine_config=None, enable_debug: bool = True,
                 enable_tracing: bool = False, host: str = "127.0.0.1", port: int = 8082,
                 tensor_parallel_shards: Optional[int] = None, pipeline_parallel_stages: Optional[int] = None,
                 gpu_ids: Optional[List[int]] = None, extra_env: Optional[Dict[str, str]] = None,
                 api_key: Optional[str] = None, embedding_model: Optional[str] = None) -> None:
        self.model, self.device, self.model_lib, self.mode = model, device, model_lib, mode
        self.engine_config = engine_config
        self.enable_debug, self.enable_tracing = enable_debug, enable_tracing
        self.host, self.port = host, port
        self.tensor_parallel_shards = tensor_parallel_shards
        self.pipeline_parallel_stages = pipeline_parallel_stages
        self.gpu_ids = gpu_ids
        self.extra_env = dict(extra_env or {})
        self.api_key = api_key
        self.embedding_model = embedding_model  # served beside the chat model on /v1/embeddings
        self._proc: Optional[subprocess.Popen] = None

    @property
    def base_url(self) -> str:
        return f"http://{self.host}:{self.port}"

    def command(self) -> List[str]:
        cmd = [sys.executable, "-m", "mlc_llm_b200", "serve", self.model, "--device", self.device,
               "--mode", self.mode, "--host", self.host, "--port", str(self.port)]
        if self.model_lib is not None:
            cmd += ["--model-lib", self.model_lib]
        if self.enable_debug:
            cmd.append("--enable-debug")
        if self.enable_tracing:
            cmd.append("--enable-tracing")
        if self.api_key:
            cmd += ["--api-key", self.api_key]
        if self.embedding_model:
            cmd += ["--embedding-model", self.embedding_model]
        overrides = []
        if self.engine_config is not None:
            for key, value in dataclasses.asdict(self.engine_config).items():
                if value is None or key in ("model", "model_lib", "mode", "additional_models", "verbose"):
                    continue
                if key in ("speculative_mode", "prefix_cache_mode", "prefill_mode"):
                    cmd += ["--" + key.replace("_", "-"), str(value)]
                elif key in _OVERRIDE_KEYS:
                    overrides.append(f"{key}={value}")
        if self.tensor_parallel_shards is not None:
            overrides.append(f"tensor_parallel_shards={self.tensor_parallel_shards}")
        if self.pipeline_parallel_stages is not None:
            overrides.append(f"pipeline_parallel_stages={self.pipeline_parallel_stages}")
        if overrides:
            cmd += ["--overrides", ";".join(overrides)]
        return cmd

    def start(self, timeout: float = 600.0, log_path: Optional[str] = None) -> None:
        env = os.environ.copy()
        env.update(self.extra_env)
        if self.gpu_ids is not None:
            env["CUDA_VISIBLE_DEVICES"] = ",".join(str(g) for g in self.gpu_ids)
        out = open(log_path, "wb") if log_path else subprocess.DEVNULL  # pylint: disable=consider-using-with
        self._proc = subprocess.Popen(self.command(), env=env, stdout=out, stderr=subprocess.STDOUT)
        deadline = time.monotonic() + timeout
        while time.monotonic() < deadline:
            if self._proc.poll() is not None:
                raise RuntimeError(f"server process exited with code {self._proc.returncode} during start-up")
            try:
                headers = {"Authorization": f"Bearer {self.api_key}"} if self.api_key else {}
                if requests.get(self.base_url + "/v1/models", timeout=2, headers=headers).status_code == 200:
                    return
            except requests.RequestException:
                pass
            time.sleep(0.25)
        self.terminate()
        raise RuntimeError(f"server did not come up within {timeout} s")

    def terminate(self) -> None:
        """Stop exactly the child this object started."""
        proc, self._proc = self._proc, None
        if proc is None or proc.poll() is not None:
            return
        proc.terminate()
        try:
            proc.wait(timeout=15)
        except subprocess.TimeoutExpired:
            proc.kill()
            proc.wait(timeout=15)

    def __enter__(self) -> "PopenServer":
        self.start()
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        self.terminate()
