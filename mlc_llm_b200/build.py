"""In-tree build of the native parts.

Two shared objects are produced next to the Python sources:

* ``mlc_llm_b200/lib/libmlcb200_kernels.so`` -- every CUDA kernel, compiled by nvcc for sm_100a only
  and exported through a plain C ABI (loaded with ctypes, see ``ops/_lib.py``);
* ``mlc_llm_b200/_core.<abi>.so`` -- the C++ serving runtime (scheduler, paged KV manager, radix
  prefix cache, samplers, streamers, JSON FFI ...) bound with pybind11.

Objects are rebuilt only when a source or header is newer than the object, so calling
:func:`build_all` at import time is cheap.  ``python -m mlc_llm_b200.build`` forces a check.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path
from typing import List

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
OBJ_DIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC,-fvisibility=hidden",
    "-Xptxas",
    "-v",
]


if os.environ.get("MLCB_GEMM_TRACE") == "1":  # per-role timestamps of the GEMM kernel (profiling builds only)
    NVCC_FLAGS.append("-DMLCB_GEMM_TRACE")


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _newer(src: Path, deps: List[Path], out: Path) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *deps])


def _run(cmd: List[str], log: Path) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.write_text(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed ({' '.join(cmd)}):\n{proc.stdout[-8000:]}")


def _dynamic_stdcxx() -> List[str]:
    """Link against the system's shared libstdc++ explicitly. Some toolchains default to the static
    archive, which would export a second copy of the C++ runtime's unique symbols into the process
    and break other extension modules (PyTorch among them)."""
    for cand in ("/usr/lib/x86_64-linux-gnu/libstdc++.so.6", "/usr/lib64/libstdc++.so.6"):
        if os.path.exists(cand):
            return [cand]
    return []


def kernels_lib_path() -> Path:
    return LIB_DIR / "libmlcb200_kernels.so"


def build_kernels(verbose: bool = False) -> Path:
    src_dir = CSRC / "kernels"
    sources = sorted(src_dir.glob("*.cu"))
    headers = sorted(src_dir.glob("*.cuh")) + sorted(src_dir.glob("*.h"))
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    out = kernels_lib_path()
    objs, jobs = [], []
    for s in sources:
        o = OBJ_DIR / (s.stem + ".o")
        objs.append(o)
        if _newer(s, headers, o):
            jobs.append((s, o))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = [
                ex.submit(
                    _run,
                    [_nvcc(), *NVCC_FLAGS, "-I", str(src_dir), "-c", str(s), "-o", str(o)],
                    OBJ_DIR / (s.stem + ".log"),
                )
                for s, o in jobs
            ]
            for f in futs:
                f.result()
        if verbose:
            for s, _ in jobs:
                print((OBJ_DIR / (s.stem + ".log")).read_text())
    if jobs or not out.exists():
        _run(
            [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-lcudart",
             *[a for f in _dynamic_stdcxx() for a in ("-Xlinker", f)]],
            OBJ_DIR / "link_kernels.log",
        )
    return out


def core_lib_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return ROOT / f"_core{suffix}"


def build_core(verbose: bool = False) -> Path:
    import pybind11  # pylint: disable=import-outside-toplevel

    src_dir = CSRC / "serve"
    sources = sorted(src_dir.glob("*.cc"))
    headers = sorted(src_dir.glob("*.h"))
    if not sources:
        raise RuntimeError(f"no C++ sources under {src_dir}")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    out = core_lib_path()
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    flags = [
        "-O2",
        "-std=c++17",
        "-fPIC",
        "-fvisibility=hidden",
        "-Wall",
        "-Wno-sign-compare",
        "-pthread",
        "-I",
        pybind11.get_include(),
        "-I",
        sysconfig.get_paths()["include"],
        "-I",
        str(src_dir),
    ]
    objs, jobs = [], []
    for s in sources:
        o = OBJ_DIR / ("core_" + s.stem + ".o")
        objs.append(o)
        if _newer(s, headers, o):
            jobs.append((s, o))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = [
                ex.submit(_run, [cxx, *flags, "-c", str(s), "-o", str(o)], OBJ_DIR / (o.stem + ".log"))
                for s, o in jobs
            ]
            for f in futs:
                f.result()
    if jobs or not out.exists():
        _run([cxx, "-shared", "-pthread", "-o", str(out), *map(str, objs), *_dynamic_stdcxx()],
             OBJ_DIR / "link_core.log")
    if verbose:
        print(f"built {out}")
    return out


def build_selftest(sanitizer: str = "") -> Path:
    """The native runtime (everything of ``csrc/serve`` except the Python bindings) linked with
    ``csrc/selftest/runtime_selftest.cc`` into a stand-alone program, optionally under a sanitizer:
    ``"address"`` (AddressSanitizer + UndefinedBehaviorSanitizer), ``"thread"`` (ThreadSanitizer) or ``""``."""
    if sanitizer not in ("", "address", "thread"):
        raise ValueError(f"unknown sanitizer {sanitizer!r}")
    src_dir = CSRC / "serve"
    sources = [s for s in sorted(src_dir.glob("*.cc")) if s.name != "bindings.cc"]
    sources.append(CSRC / "selftest" / "runtime_selftest.cc")
    headers = sorted(src_dir.glob("*.h"))
    tag = sanitizer or "plain"
    obj_dir = OBJ_DIR / f"selftest_{tag}"
    obj_dir.mkdir(parents=True, exist_ok=True)
    flags = ["-O1", "-g", "-std=c++17", "-pthread", "-fno-omit-frame-pointer", "-I", str(src_dir)]
    if sanitizer == "address":
        flags += ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]
    elif sanitizer == "thread":
        flags += ["-fsanitize=thread"]
    # not every installed g++ ships the sanitizer run-time libraries: take the first one that links a probe
    cxx = None
    probe = obj_dir / "probe.cc"
    probe.write_text("int main() { return 0; }\n")
    for cand in dict.fromkeys([os.environ.get("CXX"), "/usr/bin/g++", shutil.which("g++"), shutil.which("clang++")]):
        if not cand or not os.path.exists(cand):
            continue
        ok = subprocess.run([cand, *flags, str(probe), "-o", str(obj_dir / "probe")], capture_output=True)
        if ok.returncode == 0:
            cxx = cand
            break
    if cxx is None:
        raise FileNotFoundError(f"no C++ compiler here links with the {sanitizer or 'plain'} sanitizer run time")
    objs, jobs = [], []
    for s in sources:
        o = obj_dir / (s.stem + ".o")
        objs.append(o)
        if _newer(s, headers, o):
            jobs.append((s, o))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for f in [ex.submit(_run, [cxx, *flags, "-c", str(s), "-o", str(o)], obj_dir / (o.stem + ".log"))
                      for s, o in jobs]:
                f.result()
    out = obj_dir / "runtime_selftest"
    if jobs or not out.exists():
        _run([cxx, *flags, "-o", str(out), *map(str, objs)], obj_dir / "link.log")
    return out


def build_all(verbose: bool = False) -> None:
    build_core(verbose)
    build_kernels(verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("ok")
