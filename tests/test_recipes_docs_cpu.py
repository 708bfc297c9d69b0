"""Recipes, documents and sources as contracts: every shell recipe is run with a stand-in ``python`` that records its command
line, and the recorded overrides must compose against the shipped configs; every ``python -m pear_b200...`` command and file
the documents name exists; every module of the package imports on a machine without a GPU; every kernel launch in the CUDA
sources is followed by an error check."""

import glob
import importlib
import os
import pkgutil
import re
import stat
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _record(script: str, tmp_path, env_extra=None) -> list[list[str]]:
    """Run a recipe with ``python`` replaced by a recorder; returns the argument lists of the commands it started."""
    stub_dir = tmp_path / "bin"
    stub_dir.mkdir(exist_ok=True)
    log = tmp_path / "calls.log"
    if log.exists():
        log.unlink()
    stub = stub_dir / "python"
    stub.write_text('#!/bin/bash\nprintf "%s\\x1f" "$@" >> "$STUB_LOG"\nprintf "\\n" >> "$STUB_LOG"\n')
    stub.chmod(stub.stat().st_mode | stat.S_IEXEC)
    env = dict(os.environ, PATH=f"{stub_dir}:{os.environ['PATH']}", STUB_LOG=str(log), **(env_extra or {}))
    r = subprocess.run(["bash", script, "extra.key=1"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stderr
    return [line.split("\x1f")[:-1] for line in log.read_text().splitlines() if line]


def _compose_trainer(args: list[str]):
    from pear_b200.config.loader import compose
    from pear_b200.train.engine import EngineConfig
    from pear_b200.train.main import RunConfig

    recipe, overrides = args[0], [a for a in args[1:] if "=" in a and a != "extra.key=1"]
    cfg = RunConfig(compose(recipe, overrides)).prepare()
    EngineConfig.from_config(cfg)
    return cfg


RECIPES = sorted(glob.glob(os.path.join(ROOT, "examples", "*.sh")))


@pytest.mark.parametrize("script", RECIPES, ids=[os.path.basename(s) for s in RECIPES])
def test_recipe_overrides_compose_against_the_shipped_configs(script, tmp_path):
    variants = [{}]
    text = open(script).read()
    if "SERVE" in text:
        variants.append({"SERVE": "1"})
    if '"$N" = 1' in text:
        variants.append({"N": "1"})
    seen = 0
    if "NODE_RANK" in text:
        variants = [{"NODES": "10.0.0.1,10.0.0.2", "NODE_RANK": "0"}]
    for env in variants:
        for args in _record(script, tmp_path, {"RUN": str(tmp_path / "run"), **env}):
            helpers = ("pear_b200.rollout.server", "pear_b200.deploy.station.cli")  # started beside the program that takes the overrides
            if "-c" in args:
                continue  # a readiness probe
            if any(h in args for h in helpers):
                module = next(h for h in helpers if h in args)
                helptext = subprocess.run([sys.executable, "-m", module, "--help"], cwd=ROOT, capture_output=True, text=True, timeout=120).stdout
                for a in args[args.index(module) + 1:]:
                    if a.startswith("--"):
                        assert a in helptext, f"{os.path.basename(script)} passes {a}, which {module} does not take"
                continue
            assert args[-1] == "extra.key=1", "a recipe passes the caller's extra overrides on"
            if "pear_b200.deploy.harness.service" in args:
                from pear_b200.config.loader import compose

                rest = args[args.index("pear_b200.deploy.harness.service") + 1:]
                cfg = compose("agent_harness", [a for a in rest if a != "extra.key=1"])
                assert str(cfg.audit_dir).startswith(str(tmp_path / "run"))
                seen += 1
            elif "pear_b200.train.main" in args:
                cfg = _compose_trainer(args[args.index("pear_b200.train.main") + 1:])
                assert str(cfg.run_dir) == str(tmp_path / "run")
                seen += 1
            elif "pear_b200.launch.launch" in args:
                from pear_b200.launch.launch import main as launch_main
                from pear_b200.launch.roles import plan_node

                rest = args[args.index("pear_b200.launch.launch") + 1:]
                assert launch_main([a for a in rest if a != "extra.key=1"] + ["--dry-run"]) == 0
                flags = {rest[i]: rest[i + 1] for i in range(len(rest) - 1) if rest[i].startswith("--")}
                if "--node-addrs" in flags:
                    from pear_b200.launch.roles import plan_cluster

                    plans = {p.role: p for p in plan_cluster(flags["--node-addrs"].split(","), int(flags["--node-rank"]), int(flags.get("--gpus", 8)),
                                                             int(flags.get("--trainer-nodes", 1)), int(flags["--rollout-tp"]), rest[0],
                                                             [a for a in rest[1:] if "=" in a and a != "extra.key=1"])}
                    cfg = _compose_trainer(plans["trainer"].args)
                    assert len(cfg.actor_rollout_ref.rollout.checkpoint_engine.replica_urls) == 2  # one rollout node of 8 GPUs in replicas of 4
                    seen += 1
                    continue
                plans = {p.role: p for p in plan_node(int(flags.get("--gpus", 8)), int(flags["--trainer-gpus"]), int(flags["--rollout-tp"]), rest[0],
                                                      [a for a in rest[1:] if "=" in a and a != "extra.key=1"])}
                cfg = _compose_trainer(plans["trainer"].args)
                assert len(cfg.actor_rollout_ref.rollout.checkpoint_engine.replica_urls) == plans["rollout"].processes
                seen += 1
            elif "pear_b200.deploy.server" in args:
                from pear_b200.config.loader import compose

                rest = args[args.index("pear_b200.deploy.server") + 1:]
                compose(rest[0] if "=" not in rest[0] else "server", [a for a in rest if "=" in a and a != "extra.key=1"])
                seen += 1
            elif any(a.endswith("bench.py") for a in args):
                helptext = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True, timeout=120).stdout
                for a in args:
                    if a.startswith("--") and not a.startswith(("--nnodes", "--nproc", "--master")):
                        assert a.split("=")[0] in helptext, f"{os.path.basename(script)} passes {a}, which bench.py does not take"
                seen += 1
            else:
                raise AssertionError(f"{os.path.basename(script)} starts something this test does not know: {args[:6]}")
    assert seen >= len(variants)


def test_commands_and_files_named_by_the_documents_exist():
    # the package's own documents: the markdown files at the top whose title names the package, and the recipes' notes
    docs = [p for p in sorted(glob.glob(os.path.join(ROOT, "*.md"))) if open(p).readline().lower().startswith("# pear")]
    docs += sorted(glob.glob(os.path.join(ROOT, "examples", "*.md"))) + RECIPES
    assert len(docs) >= 3 + len(RECIPES)
    modules, paths = set(), set()
    for d in docs:
        text = open(d).read()
        modules.update(re.findall(r"python -m (pear_b200(?:\.\w+)+)", text))
        paths.update(re.findall(r"`((?:pear_b200|tests|examples|profiles)/[\w./-]+\.(?:py|cu|cuh|sh|md|yaml|h))`", text))
    assert len(modules) >= 8 and len(paths) >= 40
    for m in sorted(modules):
        mod = importlib.import_module(m)
        assert '__name__ == "__main__"' in open(mod.__file__).read(), f"`python -m {m}` is documented but the module does not run as a command"
    missing = sorted(p for p in paths if not os.path.exists(os.path.join(ROOT, p)) and not os.path.exists(os.path.join(ROOT, "pear_b200", p)))
    assert not missing, f"documents name files that do not exist: {missing}"


def test_every_module_imports_without_a_gpu():
    code = ("import importlib, pkgutil, sys, pear_b200\n"
            "bad = []\n"
            "for m in pkgutil.walk_packages(pear_b200.__path__, 'pear_b200.'):\n"
            "    if m.name.rsplit('.', 1)[-1].startswith('_pear_kernels'):\n"
            "        continue  # the kernel library is loaded through ctypes, it is not a Python module\n"
            "    try:\n"
            "        importlib.import_module(m.name)\n"
            "    except Exception as e:\n"
            "        bad.append((m.name, repr(e)))\n"
            "print(bad)\n"
            "import torch\n"
            "assert not torch.cuda.is_initialized()\n"
            "sys.exit(1 if bad else 0)\n")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


def _unchecked_launches(text: str, name: str) -> list[str]:
    unchecked = []
    lines = text.splitlines()
    for i, line in enumerate(lines):
        code = line.split("//")[0]
        if "<<<" in code:
            window = "\n".join(lines[i:i + 40])
            end = re.search(r"\n\}\s*$|\n\}\n", window)
            body = window[: end.start()] if end else window
            if "PEAR_LAUNCH_CHECK()" not in body and "cudaGetLastError" not in body:
                unchecked.append(f"{name}:{i + 1}: {code.strip()[:80]}")
        m = re.search(r"\b(launch_kernel|launch_dependent|launch_ordinary|cudaLaunchKernelEx)\s*\(", code)
        if m and not re.search(r"\b(inline|static|template)\b", code):
            prev = lines[i - 1].split("//")[0] if i else ""
            checked = re.search(r"PEAR_CUDA_CHECK\s*\(|\breturn\b|=\s*" + m.group(1), code) or re.search(r"(PEAR_CUDA_CHECK\s*\(|\breturn|=)\s*$", prev)
            if not checked:
                unchecked.append(f"{name}:{i + 1}: {code.strip()[:80]}")
    return unchecked


def test_every_kernel_launch_is_followed_by_an_error_check():
    """A ``<<<...>>>`` launch must reach ``PEAR_LAUNCH_CHECK()`` before its function ends; a launch through ``launch_kernel /
    launch_dependent / launch_ordinary / cudaLaunchKernelEx`` must have its result checked or returned."""
    good = "int f() {\n  k<<<1, 32>>>(p);\n  PEAR_LAUNCH_CHECK();\n  PEAR_CUDA_CHECK(launch_ordinary(k, g, b, 0, s, p));\n  return 0;\n}\n"
    bad = "int f() {\n  k<<<1, 32>>>(p);\n  return 0;\n}\nint g() {\n  launch_ordinary(k, g, b, 0, s, p);\n  return 0;\n}\n"
    assert _unchecked_launches(good, "good.cu") == [] and len(_unchecked_launches(bad, "bad.cu")) == 2
    unchecked = []
    for path in sorted(glob.glob(os.path.join(ROOT, "pear_b200", "ops", "csrc", "*.cu")) + glob.glob(os.path.join(ROOT, "pear_b200", "ops", "csrc", "*.cuh"))):
        unchecked += _unchecked_launches(open(path).read(), os.path.basename(path))
    assert not unchecked, "launches without an error check:\n" + "\n".join(unchecked)


def test_installation_check_runs_without_a_gpu(capsys):
    from pear_b200.utils import doctor

    rc = doctor.main([])
    out = capsys.readouterr().out
    rows = {line.split()[0] + (" " + line.split()[1] if line.split()[1] not in ("ok", "missing", "n/a") else ""): line for line in out.splitlines() if line.strip() and not line.startswith("missing:")}
    assert "GPUs" in rows and "no GPU" in rows["GPUs"] and "kernel library" in rows
    assert rc == (1 if "missing:" in out else 0)
