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


def ptr(t) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    if isinstance(t, int):
        return ctypes.c_void_p(t)
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCH_COUNT = 0  # launches of this library's kernels issued through the python bindings (bench.py reports it)


def count_launch(n: int = 1) -> None:
    global LAUNCH_COUNT
    LAUNCH_COUNT += n
