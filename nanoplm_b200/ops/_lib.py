"""ctypes loader for the in-tree sm_100a kernel libraries.

The shared objects live in ``nanoplm_b200/_lib`` (built by ``nanoplm_b200.csrc.build``). On a CUDA
machine a missing library is an error: ops never fall back silently to PyTorch on the GPU.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from nanoplm_b200.csrc import build as _build

_LOCK = threading.Lock()
_LIBS: dict[str, ctypes.CDLL] = {}
_STATUS: dict[int, torch.Tensor] = {}
_LAUNCHES = 0

STATUS_NAMES = {
    1: "a consumer waited for a TMA stage that never arrived",
    2: "the TMA producer waited for a stage that was never released",
    3: "an epilogue waited for an accumulator that never completed",
    4: "the MMA warp waited for an accumulator that was never drained",
    5: "a flag owned by another rank was never set (peer timeout)",
    6: "a bounded wait ran out",
    7: "bad argument detected on the device",
}


class KernelError(RuntimeError):
    pass


class CommTimeout(KernelError):
    """A bounded device-side wait on a peer ran out; the CUDA context is still usable."""


def lib(name: str) -> ctypes.CDLL:
    """Returns the CDLL for ``<name>.cu`` (building it first if the .so is stale or missing)."""
    with _LOCK:
        if name in _LIBS:
            return _LIBS[name]
        host = (_build.CSRC / f"{name}.cpp").exists()
        src = f"{name}.cpp" if host else f"{name}.cu"
        # build_* is a no-op when the source digest matches the stamp next to the .so and raises
        # when a rebuild is needed but fails: a library that does not match its source is never
        # loaded
        path = _build.build_host(src) if host else _build.build_one(src)
        handle = ctypes.CDLL(str(path))
        _LIBS[name] = handle
        return handle


def loaded_libraries() -> list[str]:
    return sorted(str(_build.lib_path(f"{n}.cu")) for n in _LIBS)


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels set to a non-zero code when a bounded wait runs out."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _STATUS[idx]


def check_status(device=None, reset: bool = True) -> None:
    """Synchronising read of the status word; raises KernelError / CommTimeout if set."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        if reset:
            w.zero_()
        msg = STATUS_NAMES.get(code, f"device status {code}")
        if code == 5:
            raise CommTimeout(msg)
        raise KernelError(msg)


def count_launch(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launches() -> int:
    """Number of kernels of this package launched so far in this process."""
    return _LAUNCHES


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        if rc > 0:
            raise KernelError(f"{what}: CUDA error {rc}")
        raise KernelError(f"{what}: rejected arguments (code {rc})")
