"""``python -m pear_b200.utils.doctor``: what this installation can run, checked before a job is started.

One line per item, ``ok`` / ``missing`` / ``n/a`` with the reason: the kernel library (present, built from the sources in the
tree), the compiler, the GPU generation (sm_100a or none: anything else is refused by the kernels), NCCL and symmetric memory
for the NVSwitch kernels, the host packages the roles need (FastAPI / uvicorn for replicas, aiohttp for the router, tokenizers
for model directories), the open-file limit the servers want. Upstream ships the same idea as a GPU test of its training
environment (tests/test_training_environment_on_gpu.py:37-69); here it is a command, and it runs without a GPU too.
"""

from __future__ import annotations

import importlib
import os
import shutil
import sys


def checks() -> list[tuple[str, str, str]]:
    rows: list[tuple[str, str, str]] = []

    def add(name: str, status: str, note: str = "") -> None:
        rows.append((name, status, note))

    import torch

    add("torch", "ok", f"{torch.__version__}, CUDA runtime {torch.version.cuda}")
    from ..ops import build

    nvcc = build.NVCC if os.path.exists(build.NVCC) else shutil.which("nvcc")
    add("nvcc", "ok" if nvcc else "missing", nvcc or "the kernel library cannot be rebuilt here")
    if build.LIB.exists():
        stamp = build.STAMP.read_text().strip() if build.STAMP.exists() else ""
        fresh = stamp == build.source_digest()
        add("kernel library", "ok" if fresh else "missing", str(build.LIB) if fresh else "built from other sources: run python -m pear_b200.ops.build")
    else:
        add("kernel library", "missing", "run python -m pear_b200.ops.build")
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        caps = sorted({torch.cuda.get_device_capability(i) for i in range(n)})
        good = caps == [(10, 0)]
        add("GPUs", "ok" if good else "missing", f"{n} x {torch.cuda.get_device_name(0)}, capability {caps}" + ("" if good else ": the kernels are built for sm_100a only"))
        import torch.distributed as dist

        add("NCCL", "ok" if dist.is_nccl_available() else "missing", ".".join(map(str, torch.cuda.nccl.version())) if dist.is_nccl_available() else "")
        try:
            importlib.import_module("torch.distributed._symmetric_memory")
            add("symmetric memory", "ok" if n > 1 else "n/a", "peer-memory kernels need two or more GPUs" if n < 2 else "torch.distributed._symmetric_memory")
        except ImportError as e:
            add("symmetric memory", "missing", repr(e))
        free, total = torch.cuda.mem_get_info(0)
        add("GPU memory", "ok", f"{free / 2**30:.0f} of {total / 2**30:.0f} GiB free on GPU 0")
    else:
        add("GPUs", "n/a", "no GPU: the fp32 reference ops run (CPU plumbing and tests)")
    for mod, role in (("fastapi", "replica and deploy servers"), ("uvicorn", "replica and deploy servers"), ("requests", "trainer -> replica processes"),
                      ("aiohttp", "evaluation router"), ("tokenizers", "tokenizer.json of model directories"), ("yaml", "recipes"), ("numpy", "trajectories")):
        try:
            m = importlib.import_module(mod)
            add(mod, "ok", f"{getattr(m, '__version__', '')} ({role})")
        except ImportError:
            add(mod, "missing", role)
    try:
        import resource

        soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
        add("open files", "ok" if soft >= 4096 or hard >= 4096 else "missing", f"soft {soft}, hard {hard} (servers raise the soft limit at start)")
    except (ImportError, OSError):
        add("open files", "n/a", "")
    from .process import node_cpus

    try:
        add("NUMA", "ok", f"node 0: {len(node_cpus(0))} CPUs (replicas bind to their GPU's node)")
    except OSError:
        add("NUMA", "n/a", "no /sys/devices/system/node: replicas run unbound")
    return rows


def main(argv=None) -> int:
    rows = checks()
    width = max(len(r[0]) for r in rows)
    for name, status, note in rows:
        print(f"{name:{width}s}  {status:8s} {note}")
    bad = [r[0] for r in rows if r[1] == "missing"]
    if bad:
        print(f"\nmissing: {', '.join(bad)}")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main(sys.argv[1:]))
