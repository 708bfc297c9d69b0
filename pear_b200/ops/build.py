"""Builds the in-tree CUDA library ``pear_b200/ops/_pear_kernels.so`` for sm_100a with nvcc.

Every ``csrc/*.cu`` is compiled to an object in parallel (``-gencode arch=compute_100a,code=sm_100a -lineinfo``) and
linked into one shared library with plain C entry points (loaded through ctypes by :mod:`pear_b200.ops.lib`), so a
build needs neither the torch headers nor a GPU. Objects are rebuilt only when a source or header is newer.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = HERE / "_pear_kernels.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


STAMP = HERE / "_pear_kernels.src"  # digest of the sources the library was built from (checked by the loader)


def source_digest() -> str:
    """One digest over every source and header: the loader refuses a library built from other sources (a C entry point
    whose argument list changed would otherwise be called with shifted arguments)."""
    import hashlib

    h = hashlib.sha256()
    for p in sorted([*CSRC.glob("*.cu"), *CSRC.glob("*.cuh"), *CSRC.glob("*.h")]):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _newest_header() -> float:
    return max((p.stat().st_mtime for p in [*CSRC.glob("*.cuh"), *CSRC.glob("*.h")]), default=0.0)


def build(verbose: bool = False, ptxas_info: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_time = _newest_header()
    jobs = []
    for src in sources:
        obj = BUILD / (src.stem + ".o")
        if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, header_time):
            continue
        cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, r in pool.map(run, jobs):
            if verbose or r.returncode != 0 or ptxas_info:
                sys.stderr.write(f"[nvcc] {src.name}\n{r.stdout}{r.stderr}\n")
            failed |= r.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    objs = [str(BUILD / (s.stem + ".o")) for s in sources]
    if jobs or not LIB.exists():
        cmd = [NVCC, "-shared", "-o", str(LIB), *objs, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    STAMP.write_text(source_digest())
    return LIB


def resources() -> list[dict]:
    """What the compiler made of every kernel, from ``-Xptxas -v`` (registers, spills, static shared memory, barriers): each
    source is compiled once more into a scratch object; nothing of the build is touched and no GPU is needed."""
    import re
    import tempfile

    rows: list[dict] = []

    def run(src):
        with tempfile.TemporaryDirectory() as d:
            r = subprocess.run([NVCC, "-Xptxas", "-v", *FLAGS, "-c", str(src), "-o", os.path.join(d, "x.o")], capture_output=True, text=True)
        return src, r

    with ThreadPoolExecutor(max_workers=8) as pool:
        for src, r in pool.map(run, sorted(CSRC.glob("*.cu"))):
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stderr}")
            name, spill = None, (0, 0, 0)
            for line in r.stderr.splitlines():
                m = re.search(r"Compiling entry function '(\S+)'", line)
                if m:
                    name = m.group(1)
                    continue
                m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
                if m:
                    spill = tuple(int(x) for x in m.groups())
                    continue
                m = re.search(r"Used (\d+) registers(?:, used (\d+) barriers)?(?:, (\d+) bytes smem)?", line)
                if m and name:
                    rows.append({"file": src.name, "kernel": name, "registers": int(m.group(1)), "barriers": int(m.group(2) or 0),
                                 "static_smem": int(m.group(3) or 0), "stack": spill[0], "spill_stores": spill[1], "spill_loads": spill[2]})
                    name, spill = None, (0, 0, 0)
    names = "\n".join(r["kernel"] for r in rows)
    try:  # readable names when binutils is present
        out = subprocess.run(["c++filt"], input=names, capture_output=True, text=True, check=True).stdout.splitlines()
        for r, n in zip(rows, out):
            r["kernel"] = re.sub(r"\(.*$", "", n).replace("pear::", "").replace("(anonymous namespace)::", "")
    except (OSError, subprocess.CalledProcessError):
        pass
    return rows


if __name__ == "__main__":
    if "--resources" in sys.argv:
        table = resources()
        print("| file | kernel | registers | spill stores / loads (B) | stack (B) | static smem (B) | barriers |\n| --- | --- | --- | --- | --- | --- | --- |")
        for r in table:
            print(f"| {r['file']} | `{r['kernel']}` | {r['registers']} | {r['spill_stores']} / {r['spill_loads']} | {r['stack']} | {r['static_smem']} | {r['barriers']} |")
        spilled = [r for r in table if r["spill_stores"] or r["spill_loads"]]
        print(f"\n{len(table)} kernels, {len(spilled)} with register spills, at most {max(r['registers'] for r in table)} registers per thread")
    else:
        print(build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
