"""Builds the sm_100a kernels into in-tree shared objects with plain nvcc.

Each ``.cu`` file becomes ``nanoplm_b200/_lib/lib<name>.so`` exposing a C ABI (``extern "C"``
functions taking raw device pointers and a ``cudaStream_t``); ``nanoplm_b200.ops._lib`` loads them
with ctypes. nvcc cross-compiles without a GPU, so the build also works on a CPU-only machine.

Run ``python -m nanoplm_b200.csrc.build`` (add ``-v`` for ptxas register / shared-memory usage).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_DIR = CSRC.parent / "_lib"

SOURCES = [
    "gemm_tcgen05.cu",
    "elementwise.cu",
    "attention.cu",
    "attention_ws.cu",
    "attention_bias.cu",
    "extras.cu",
    "comm.cu",
    "moe.cu",
    "fp8.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-shared",
]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def lib_path(name: str) -> Path:
    return LIB_DIR / f"lib{Path(name).stem}.so"


def _locked_build(out: Path, digest: str, cmd: list[str], what: str, verbose: bool, force: bool) -> Path:
    """Runs `cmd` (which writes to the path after its ``-o``) under an inter-process file lock, into a
    temporary name that is renamed into place; the digest stamp is written last. Concurrent ranks /
    DataLoader workers that see a stale stamp therefore either build once or wait, and nobody can
    dlopen a half-written library."""
    import fcntl
    stamp = out.with_suffix(".sha")
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    with open(LIB_DIR / f".{out.stem}.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
                return out   # another process built it while we waited
            tmp = out.with_name(f".{out.name}.{os.getpid()}.tmp")
            full = [tmp.as_posix() if c == "@OUT@" else c for c in cmd]
            proc = subprocess.run(full, capture_output=True, text=True)
            if proc.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise RuntimeError(f"build failed for {what}:\n{proc.stdout}\n{proc.stderr}")
            if verbose:
                sys.stderr.write(proc.stderr)
            stamp.unlink(missing_ok=True)      # never leave a matching stamp beside an old library
            os.replace(tmp, out)
            stamp.write_text(digest)
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def build_one(name: str, verbose: bool = False, force: bool = False) -> Path:
    src = CSRC / name
    out = lib_path(name)
    stamp = out.with_suffix(".sha")
    digest = _digest(src)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    cmd = [nvcc_path(), *NVCC_FLAGS, "-I", str(CSRC), "-o", "@OUT@", str(src)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    return _locked_build(out, digest, cmd, name, verbose, force)


HOST_SOURCES = ["packer.cpp"]


def build_host(name: str, force: bool = False) -> Path:
    """Builds a host-only C++ source (no CUDA) with g++."""
    src = CSRC / name
    out = lib_path(name)
    stamp = out.with_suffix(".sha")
    digest = hashlib.sha256(src.read_bytes()).hexdigest()
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-o", "@OUT@", str(src)]
    return _locked_build(out, digest, cmd, name, False, force)


def build_all(verbose: bool = False, force: bool = False) -> list[Path]:
    names = [n for n in SOURCES if (CSRC / n).exists()]
    with ThreadPoolExecutor(max_workers=min(8, len(names))) as ex:
        libs = list(ex.map(lambda n: build_one(n, verbose, force), names))
    libs += [build_host(n, force) for n in HOST_SOURCES if (CSRC / n).exists()]
    return libs


if __name__ == "__main__":
    v = "-v" in sys.argv
    f = "-f" in sys.argv
    for p in build_all(verbose=v, force=f):
        print(p)
