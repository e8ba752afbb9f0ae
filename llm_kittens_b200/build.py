"""In-tree build of the native libraries.

Two shared objects are produced under ``llm_kittens_b200/_lib``:

* ``libllmk_cuda.so``  - every hand-written sm_100a kernel (``csrc/*.cu``), compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a``; plain C ABI, loaded with ctypes.
* ``libllmk_host.so``  - host runtime in C++ (``csrc/host/*.cpp``): token-shard data loader, eval
  loader, tokenizer, torch-compatible mt19937 random init, checkpoint streaming.

Objects are rebuilt only when a source or header is newer than the object, so calling ``build()``
from tests or from the command line is cheap when nothing changed:

    python -m llm_kittens_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "_lib"
OBJDIR = LIBDIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA kernels of llm_kittens_b200 cannot be built")
    return cand


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _run(cmd, verbose: bool, log: Path | None = None) -> None:
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(map(str, cmd)) + "\n" + res.stdout)
    if verbose:
        print(res.stdout)


def cuda_lib_path() -> Path:
    return LIBDIR / "libllmk_cuda.so"


def host_lib_path() -> Path:
    return LIBDIR / "libllmk_host.so"


def build(force: bool = False, verbose: bool = False) -> None:
    """Compile what is out of date. Raises RuntimeError with the compiler output on failure."""
    OBJDIR.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((CSRC / "host").glob("*.h"))
    hdr_time = _newest(headers)

    # ---- CUDA kernels
    cu_sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    objs = []
    for src in cu_sources:
        obj = OBJDIR / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            jobs.append((cmd, OBJDIR / (src.stem + ".ptxas.log")))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(j[0], verbose, j[1]), jobs))
    lib = cuda_lib_path()
    if cu_sources and (force or jobs or not lib.exists()):
        _run([_nvcc(), "-shared", "-o", str(lib), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
              "-cudart", "static"], verbose)

    # ---- host runtime
    cpp_sources = sorted((CSRC / "host").glob("*.cpp"))
    hlib = host_lib_path()
    if cpp_sources and (force or not hlib.exists() or hlib.stat().st_mtime < max(_newest(cpp_sources), hdr_time)):
        _run(["g++", *CXX_FLAGS, "-shared", "-o", str(hlib), *map(str, cpp_sources), "-I", str(CSRC / "host")], verbose)


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel as printed by ``ptxas -v`` at the last build."""
    out = []
    for log in sorted(OBJDIR.glob("*.ptxas.log")):
        out.append(f"== {log.stem}")
        out.append(log.read_text())
    return "\n".join(out)


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print("built:", cuda_lib_path(), host_lib_path())
