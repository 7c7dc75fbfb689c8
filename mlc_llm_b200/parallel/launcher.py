"""Start the worker ranks of a multi-GPU engine from the serving process.

The serving process becomes rank 0; ranks 1..N-1 are child processes running
``python -m mlc_llm_b200.cli.worker`` with the usual ``RANK`` / ``WORLD_SIZE`` / ``MASTER_*``
environment (reference: Disco ``ProcessSession`` spawning ``mlc_llm.cli.worker``,
``cpp/serve/engine.cc:872-877``, ``python/mlc_llm/cli/worker.py:29-50``).  Under ``torchrun`` the
ranks already exist and nothing is spawned.
"""

from __future__ import annotations

import atexit
import json
import os
import socket
import subprocess
import sys
from typing import List, Optional

import torch

from . import Communicator


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class WorkerGroup:
    """Child processes of ranks 1..N-1 plus rank 0's communicator."""

    def __init__(self, comm: Communicator, procs: List[subprocess.Popen]):
        self.comm = comm
        self.procs = procs
        atexit.register(self.shutdown)

    def shutdown(self) -> None:
        procs, self.procs = self.procs, []
        if procs:
            try:
                self.comm.shutdown_workers()
            except Exception:  # pylint: disable=broad-except
                pass
        for p in procs:
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                p.kill()
        if procs:
            self.comm.destroy()


def launch(engine_config, device: torch.device, tp: int, pp: int = 1,
           timeout_s: float = 600.0) -> Optional[WorkerGroup]:
    """Returns the group for rank 0, or None when a single process is enough."""
    world = tp * pp
    if world <= 1:
        return None
    if "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) == world:
        return WorkerGroup(Communicator(tp, pp, timeout_s=timeout_s), [])
    port = _free_port()
    base = os.environ.copy()
    base.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "WORLD_SIZE": str(world)})
    cfg_json = engine_config.asjson()
    procs = []
    for rank in range(1, world):
        env = dict(base)
        env.update({"RANK": str(rank), "LOCAL_RANK": str(rank)})
        procs.append(subprocess.Popen(  # pylint: disable=consider-using-with
            [sys.executable, "-m", "mlc_llm_b200.cli.worker", "--engine-config", cfg_json,
             "--device", device.type, "--tp", str(tp), "--pp", str(pp)], env=env))
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "WORLD_SIZE": str(world),
                       "RANK": "0", "LOCAL_RANK": "0"})
    dev = torch.device("cuda", 0) if device.type == "cuda" else device
    comm = Communicator(tp, pp, device=dev, timeout_s=timeout_s)
    return WorkerGroup(comm, procs)


def worker_main(argv=None) -> None:
    """Entry of a spawned worker rank."""
    import argparse  # pylint: disable=import-outside-toplevel

    from ..serve.config import EngineConfig  # pylint: disable=import-outside-toplevel
    from ..serve.engine_base import EngineRuntime  # pylint: disable=import-outside-toplevel
    from . import env_world, worker_loop  # pylint: disable=import-outside-toplevel

    ap = argparse.ArgumentParser("mlc_llm_b200 worker rank")
    ap.add_argument("--engine-config", required=True)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--tp", type=int, required=True)
    ap.add_argument("--pp", type=int, default=1)
    args = ap.parse_args(argv)
    _, _, local = env_world()
    dev = torch.device("cuda", local) if args.device == "cuda" else torch.device("cpu")
    comm = Communicator(args.tp, args.pp, device=dev)
    cfg = EngineConfig.from_json(args.engine_config)
    _ = json
    runtime = EngineRuntime(cfg, dev, comm=comm)
    try:
        worker_loop(runtime.executor, comm)
    finally:
        comm.destroy()
