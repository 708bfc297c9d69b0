"""Layering and hygiene: the generic runtime never names a model family, nothing imports scratch code, and every CUDA
source names no closed call."""

import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parent.parent
PKG = ROOT / "pear_b200"
GENERIC = ["train", "rollout", "loop", "sim", "envs", "monitor", "eval", "parallel", "utils", "launch", "config"]


def test_generic_runtime_does_not_import_a_model_family():
    pat = re.compile(r"^\s*(from|import)\s+[\w.]*qwen3_5", re.M)
    offenders = [str(p.relative_to(ROOT)) for d in GENERIC for p in (PKG / d).rglob("*.py") if pat.search(p.read_text())]
    assert not offenders, offenders


def test_nothing_committed_uses_scratch_code():
    pat = re.compile(r"(from|import)\s+_work|[\"']_work/")
    offenders = [str(p.relative_to(ROOT)) for p in list(PKG.rglob("*.py")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"] if pat.search(p.read_text())]
    assert not offenders, offenders


def test_cuda_sources_avoid_closed_calls_and_multicast_loads():
    # (the patterns are assembled from pieces so that this file itself does not contain the strings it looks for)
    bad = re.compile("|".join(["Memcpy" + "BatchAsync", "Memcpy3D" + "BatchAsync", r"cp\.async\.bulk[\w.:]*multi" + "cast::" + "cluster"]))
    offenders = [p.name for p in (PKG / "ops" / "csrc").glob("*.cu*") if bad.search(p.read_text())]
    assert not offenders, offenders


def test_every_device_wait_in_the_peer_kernels_is_bounded():
    src = (PKG / "ops" / "csrc" / "comm_kernels.cu").read_text() + (PKG / "ops" / "csrc" / "gemm_collective.cu").read_text()
    assert "while (true)" not in src and "while(1)" not in src and "for (;;)" not in src
    assert "__trap" not in src
