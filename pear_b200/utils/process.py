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


def free_ports(n: int, host: str = "127.0.0.1") -> list[int]:
    """``n`` DISTINCT free ports: all sockets stay open until every port is known (two calls of ``free_port`` in a row may be
    handed the same port)."""
    socks = []
    try:
        for _ in range(n):
            s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            s.bind((host, 0))
            socks.append(s)
        return [s.getsockname()[1] for s in socks]
    finally:
        for s in socks:
            s.close()


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


_SYS_SET_MEMPOLICY, _SYS_MOVE_PAGES = 238, 279  # x86_64 system call numbers
_MPOL_PREFERRED = 1


def node_cpus(node: int) -> list[int]:
    """CPUs of a NUMA node from sysfs (``0-7,16-23`` notation)."""
    with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
        text = f.read().strip()
    cpus: list[int] = []
    for part in filter(None, text.split(",")):
        lo, _, hi = part.partition("-")
        cpus += list(range(int(lo), int(hi or lo) + 1))
    return cpus


def set_numa_affinity(node: int) -> bool:
    """Run this process on the CPUs of ``node`` and prefer its memory for what it allocates from now on (pinned host buffers
    land on the node of the thread that first touches them). Plain system calls (``sched_setaffinity``, ``set_mempolicy``), so
    no libnuma is needed (upstream binds its cache sidecar with ``numactl --cpunodebind --membind``:
    pear/rollout/lmcache.py:21-221). False when the platform refuses or has no such node."""
    import platform

    try:
        cpus = node_cpus(node)
        if not cpus:
            return False
        os.sched_setaffinity(0, cpus)
        if platform.machine() != "x86_64":
            return True  # CPU binding only: first touch then places the memory
        libc = ctypes.CDLL(ctypes.util.find_library("c") or "libc.so.6", use_errno=True)
        libc.syscall.restype = ctypes.c_long
        words = node // 64 + 1
        mask = (ctypes.c_ulong * words)()
        mask[node // 64] = 1 << (node % 64)
        rc = libc.syscall(ctypes.c_long(_SYS_SET_MEMPOLICY), ctypes.c_int(_MPOL_PREFERRED), ctypes.byref(mask), ctypes.c_ulong(64 * words + 1))
        return rc == 0
    except (OSError, ValueError):
        return False


def numa_locality(address: int, nbytes: int, node: int, samples: int = 512, page: int = 4096) -> Optional[float]:
    """Fraction of (sampled) resident pages of ``[address, address + nbytes)`` that sit on ``node``, from the ``move_pages``
    query form; None when the platform does not answer. Upstream waits until its host tier is >= 95 % local to the GPUs' node."""
    import platform

    if platform.machine() != "x86_64" or nbytes <= 0:
        return None
    try:
        libc = ctypes.CDLL(ctypes.util.find_library("c") or "libc.so.6", use_errno=True)
        libc.syscall.restype = ctypes.c_long
        n_pages = max(1, nbytes // page)
        count = min(samples, n_pages)
        first = address - address % page
        pages = (ctypes.c_void_p * count)(*[first + (i * n_pages // count) * page for i in range(count)])
        status = (ctypes.c_int * count)()
        rc = libc.syscall(ctypes.c_long(_SYS_MOVE_PAGES), ctypes.c_int(0), ctypes.c_ulong(count), pages, None, status, ctypes.c_int(0))
        if rc != 0:
            return None
        resident = [s for s in status if s >= 0]
        return (sum(s == node for s in resident) / len(resident)) if resident else None
    except OSError:
        return None


def visible_gpu_index(local_index: int = 0) -> int:
    """The machine-wide index of this process's ``local_index``-th GPU (``CUDA_VISIBLE_DEVICES`` renumbers them)."""
    vis = [v for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
    try:
        return int(vis[local_index]) if vis else local_index
    except (ValueError, IndexError):
        return local_index


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
