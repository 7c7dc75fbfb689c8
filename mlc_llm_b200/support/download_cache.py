"""Model download cache: ``HF://org/repo`` and ``https://huggingface.co/org/repo`` resolve to
``$MLC_LLM_HOME/model_weights/hf/org/repo`` and are fetched with ``git clone`` + per-shard downloads
verified by the md5 sums of ``tensor-cache.json`` (reference:
``python/mlc_llm/support/download_cache.py:30-250``).  Cache policy comes from
``MLC_DOWNLOAD_CACHE_POLICY``: ``ON`` (use or fill), ``REDO`` (always refetch), ``READONLY`` (use,
never fetch), ``OFF`` (no caching: fetch into a temporary directory)."""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Optional, Tuple

from . import constants

HF_PREFIXES = ("HF://", "https://huggingface.co/")


def split_repo(model_url: str) -> Tuple[str, str]:
    for pre in HF_PREFIXES:
        if model_url.startswith(pre):
            rest = model_url[len(pre):].strip("/")
            parts = rest.split("/")
            if len(parts) < 2:
                raise ValueError(f"{model_url}: expected HF://<user>/<repo>")
            return parts[0], parts[1]
    raise ValueError(f"{model_url}: not a HuggingFace model reference")


def _md5(path: Path) -> str:
    h = hashlib.md5()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def _verify(model_dir: Path) -> List[str]:
    """Names of shard files that are missing or whose md5 does not match."""
    cache = model_dir / "tensor-cache.json"
    if not cache.exists():
        cache = model_dir / "ndarray-cache.json"
    if not cache.exists():
        return []
    with open(cache, encoding="utf-8") as f:
        doc = json.load(f)
    bad = []
    for shard in doc.get("records", []):
        p = model_dir / shard["dataPath"]
        if not p.exists() or ("md5sum" in shard and _md5(p) != shard["md5sum"]):
            bad.append(shard["dataPath"])
    return bad


def _run(cmd: List[str], cwd: Optional[Path] = None, env=None) -> None:
    subprocess.run(cmd, cwd=cwd, env=env, check=True, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)


def _fetch(user: str, repo: str, dest: Path, workers: int = 4) -> None:
    """``git clone`` without LFS payloads, then fetch each shard over HTTPS and verify it."""
    url = f"https://huggingface.co/{user}/{repo}"
    env = dict(os.environ, GIT_LFS_SKIP_SMUDGE="1")
    with tempfile.TemporaryDirectory(dir=constants.MLC_TEMP_DIR) as tmp:
        clone = Path(tmp) / "clone"
        try:
            _run(["git", "clone", url, str(clone)], env=env)
        except (subprocess.CalledProcessError, FileNotFoundError) as err:
            raise RuntimeError(f"cannot download {url} (no network access or git missing): {err}") from err
        cache = clone / "tensor-cache.json"
        if not cache.exists():
            cache = clone / "ndarray-cache.json"
        shards = []
        if cache.exists():
            with open(cache, encoding="utf-8") as f:
                shards = [(s["dataPath"], s.get("md5sum")) for s in json.load(f)["records"]]

        def pull(item):
            name, md5 = item
            target = clone / name
            import requests  # pylint: disable=import-outside-toplevel

            with requests.get(f"{url}/resolve/main/{name}", stream=True, timeout=60) as r:
                r.raise_for_status()
                with open(target, "wb") as out:
                    for chunk in r.iter_content(1 << 20):
                        out.write(chunk)
            if md5 and _md5(target) != md5:
                raise RuntimeError(f"md5 mismatch for {name}")

        with ThreadPoolExecutor(max_workers=workers) as pool:
            list(pool.map(pull, shards))
        shutil.rmtree(clone / ".git", ignore_errors=True)
        dest.parent.mkdir(parents=True, exist_ok=True)
        if dest.exists():
            shutil.rmtree(dest)
        shutil.move(str(clone), str(dest))


def get_or_download_model(model: str) -> Path:
    user, repo = split_repo(model)
    policy = constants.MLC_DOWNLOAD_CACHE_POLICY
    readonly = constants.MLC_LLM_READONLY_WEIGHT_CACHE
    if readonly:
        for base in readonly.split(os.pathsep):
            cand = Path(base) / "model_weights" / "hf" / user / repo
            if (cand / "mlc-chat-config.json").exists():
                return cand
    dest = constants.MLC_LLM_HOME / "model_weights" / "hf" / user / repo
    if policy == "OFF":
        dest = Path(tempfile.mkdtemp(dir=constants.MLC_TEMP_DIR)) / repo
    if policy in ("ON", "READONLY") and (dest / "mlc-chat-config.json").exists() and not _verify(dest):
        return dest
    if policy == "READONLY":
        raise RuntimeError(f"{model} is not in the cache ({dest}) and MLC_DOWNLOAD_CACHE_POLICY=READONLY")
    _fetch(user, repo, dest)
    return dest
