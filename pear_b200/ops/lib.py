"""ctypes loader of the in-tree CUDA library ``_pear_kernels.so`` (built by :mod:`pear_b200.ops.build`).

On a machine with a GPU the library MUST load: :func:`lib` raises instead of letting callers fall back to eager torch,
so a GPU test can never pass on a silent fallback. Entry points are plain C (``extern "C"``) taking device pointers and
a stream handle; every launcher returns a ``cudaError_t`` (0 = success) that :func:`check` turns into an exception.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB = None
LIB_PATH = Path(__file__).resolve().parent / "_pear_kernels.so"


class KernelLibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            if os.environ.get("PEAR_B200_BUILD_ON_IMPORT", "0") == "1":
                from .build import build

                build()
            else:
                raise KernelLibraryMissing(
                    f"{LIB_PATH} is missing: run `python -m pear_b200.ops.build` (nvcc cross-compiles without a GPU)")
        from .build import STAMP, source_digest

        if not STAMP.exists() or STAMP.read_text().strip() != source_digest():
            raise KernelLibraryMissing(
                f"{LIB_PATH} was built from other sources than those in csrc/: run `python -m pear_b200.ops.build`")
        _LIB = ctypes.CDLL(str(LIB_PATH))
    return _LIB


def available() -> bool:
    return LIB_PATH.exists()


def check(code: int, what: str = "kernel launch") -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with CUDA error {code}")


def expect(dtype: torch.dtype, _contiguous: bool = True, **tensors) -> None:
    """The kernels take raw pointers: a tensor of another element type (or a strided view where the kernel takes no stride)
    would be read past its end. Raise instead (``None`` entries are optional arguments)."""
    for name, t in tensors.items():
        if t is None:
            continue
        if t.dtype != dtype:
            raise TypeError(f"{name}: the kernel reads {dtype}, got {t.dtype}")
        if _contiguous and not t.is_contiguous():
            raise ValueError(f"{name}: the kernel needs a contiguous tensor")


def ptr(t) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    if isinstance(t, int):
        return ctypes.c_void_p(t)
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    """The current stream of the calling thread's current device: the kernels launch there, so a thread that works on another
    GPU than device 0 must have called ``torch.cuda.set_device`` (see :func:`on_device`)."""
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def on_device(t: torch.Tensor) -> None:
    """Raise when ``t`` lives on another GPU than the calling thread's current device (host threads start on device 0)."""
    if t.is_cuda and t.device.index != torch.cuda.current_device():
        raise RuntimeError(f"tensor on cuda:{t.device.index} but this thread's current device is cuda:{torch.cuda.current_device()}: "
                           "call torch.cuda.set_device in the thread before launching kernels")


LAUNCH_COUNT = 0  # launches of this library's kernels issued through the python bindings (bench.py reports it)


def count_launch(n: int = 1) -> None:
    global LAUNCH_COUNT
    LAUNCH_COUNT += n
