"""Process helpers: a free TCP port, dying with the parent (PR_SET_PDEATHSIG), a supervised worker process, NUMA
affinity by the GPU's node (upstream ``pear/utils``: ``free_port``, ``die_with_parent``, ``WorkerProcess``;
``3rdparty/verl/patches/0038-*`` loads libnuma by its runtime name)."""

from __future__ import annotations

import ctypes
import ctypes.util
import multiprocessing as mp
import os
import signal
import socket
from typing import Callable, Optional


def free_port(host: str = "127.0.0.1") -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return s.getsockname()[1]


def die_with_parent(sig: int = signal.SIGTERM) -> None:
    """Ask the kernel to signal this process when its parent exits (Linux prctl PR_SET_PDEATHSIG = 1)."""
    try:
        libc = ctypes.CDLL(ctypes.util.find_library("c") or "libc.so.6", use_errno=True)
        libc.prctl(1, sig)
    except OSError:
        pass


def dump_stacks_on_signal(sig: int = signal.SIGUSR1) -> None:
    """``kill -USR1 <pid>`` prints every thread's Python stack to stderr: the first question about a role process that
    stopped making progress is where it waits."""
    import faulthandler

    try:
        faulthandler.register(sig, all_threads=True, chain=False)
    except (AttributeError, ValueError, OSError):  # not on this platform / not on the main thread
        pass


def _child(target, args, kwargs):
    die_with_parent()
    target(*args, **kwargs)


class WorkerProcess:
    """A child process that dies with its parent and can be stopped with a grace period."""

    def __init__(self, target: Callable, *args, name: Optional[str] = None, **kwargs):
        ctx = mp.get_context("spawn")
        self.proc = ctx.Process(target=_child, args=(target, args, kwargs), name=name, daemon=True)

    def start(self) -> "WorkerProcess":
        self.proc.start()
        return self

    def alive(self) -> bool:
        return self.proc.is_alive()

    def stop(self, grace_s: float = 5.0) -> None:
        if self.proc.is_alive():
            self.proc.terminate()
            self.proc.join(grace_s)
        if self.proc.is_alive():
            self.proc.kill()
            self.proc.join(grace_s)


def set_numa_affinity(node: int) -> bool:
    """Bind this process's CPUs to a NUMA node through libnuma (loaded by its runtime name). False if unavailable."""
    for name in ("libnuma.so.1", "libnuma.so"):
        try:
            numa = ctypes.CDLL(name)
        except OSError:
            continue
        if numa.numa_available() < 0:
            return False
        numa.numa_run_on_node(ctypes.c_int(node))
        numa.numa_set_preferred(ctypes.c_int(node))
        return True
    return False


def gpu_numa_node(gpu_index: int) -> Optional[int]:
    """NUMA node of a GPU from sysfs (None when the platform does not expose it)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(gpu_index)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:
            bus = bus[4:]
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            n = int(f.read().strip())
        return n if n >= 0 else None
    except Exception:  # noqa: BLE001
        return None
