"""In-tree build of the native libraries.

Two shared objects are produced next to the sources (git-ignored, shipped with the tree):

* ``lib/librembrandt_cuda.so`` -- every ``csrc/*.cu`` kernel file, compiled by ``nvcc`` for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``) and linked against the static CUDA runtime so that the
  library loads on machines without a GPU (nothing touches the driver until a kernel is launched).
* ``lib/librembrandt_host.so`` -- the CPU-only runtime pieces (``csrc/host/*.cc``): NdArray blob codec,
  IDX / CIFAR readers, xorshift128+ RNG, partition helpers.

Both are bound through ``ctypes`` (see ``_native.py``); there is no torch C++ ABI dependency.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "lib"
OBJDIR = CSRC / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
# --use_fast_math (approximate division / square root, flush-to-zero) only where no statistic, normaliser or loss is
# computed: the tensor-core kernel's epilogue, pooling, data movement. Softmax / cross-entropy, LRN, batch-norm, the
# optimizer and the exchange kernels that apply it are compiled with IEEE division and square root; where they call
# an intrinsic such as __expf they do so explicitly.
PRECISE_SOURCES = {"softmax_ce.cu", "lrn.cu", "bn.cu", "sgd_fused.cu", "comm_p2p.cu"}
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return cand


def _newer(src: Path, dst: Path, extra: list[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *extra])


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build_cuda(force: bool = False, verbose: bool = False, defines: tuple = ()) -> Path:
    """`defines` (e.g. ("RB_GEMM_PROFILE",)) are passed as -D to every kernel file and force a rebuild; a library
    built with them should be rebuilt without them afterwards (`python -m rembrandt_b200._build --force`)."""
    LIBDIR.mkdir(exist_ok=True)
    OBJDIR.mkdir(exist_ok=True)
    out = LIBDIR / "librembrandt_cuda.so"
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    force = force or bool(defines)
    for src in sources:
        obj = OBJDIR / (src.stem + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            fast = [] if src.name in PRECISE_SOURCES else ["--use_fast_math"]
            cmd = [nvcc, *NVCC_FLAGS, *fast, *(f"-D{d}" for d in defines), "-I", str(CSRC), "-c", str(src), "-o",
                   str(obj)]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    if force or jobs or not out.exists():
        _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-cudart", "static", "-lpthread", "-ldl", "-lrt"])
    return out


def build_host(force: bool = False) -> Path:
    LIBDIR.mkdir(exist_ok=True)
    OBJDIR.mkdir(exist_ok=True)
    out = LIBDIR / "librembrandt_host.so"
    hdir = CSRC / "host"
    headers = sorted(hdir.glob("*.h"))
    sources = sorted(hdir.glob("*.cc"))
    cxx = shutil.which("g++") or "g++"
    objs = []
    rebuilt = False
    for src in sources:
        obj = OBJDIR / ("host_" + src.stem + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            _run([cxx, *CXX_FLAGS, "-I", str(hdir), "-c", str(src), "-o", str(obj)])
            rebuilt = True
    if force or rebuilt or not out.exists():
        _run([cxx, "-shared", "-o", str(out), *map(str, objs), "-pthread"])
    return out


def build_all(force: bool = False, verbose: bool = False, defines: tuple = ()) -> None:
    build_host(force)
    build_cuda(force, verbose, defines)


if __name__ == "__main__":
    # --profile: the tensor-core kernel counts the cycles its roles spend waiting (read by `bench_conv --roles`)
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv,
              defines=("RB_GEMM_PROFILE",) if "--profile" in sys.argv else ())
    print("built:", *(str(p) for p in sorted(LIBDIR.glob("*.so"))))
