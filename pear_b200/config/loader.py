"""Recipe/config system: YAML files composed with ``defaults`` lists, ``+group=name`` family overlays, dotted
``key=value`` overrides, ``${path}`` interpolation and ``???`` required values.

It keeps the upstream key names (``pear/configs/base.yaml``, ``training.yaml``, ``pear/models/qwen3_5/config.yaml``):
``run_dir``, ``run_sizes.*``, ``algorithm.*``, ``trainer.*``, ``data.*``, ``actor_rollout_ref.{model,actor,rollout}.*``,
so an upstream recipe's override list is accepted as is. It is a small stand-alone composer (no Hydra/OmegaConf in the
image); plug-ins are named by class path strings and resolved with :func:`load_class`.
"""

from __future__ import annotations

import copy
import importlib
import os
import re
from pathlib import Path
from typing import Any

import yaml

CONFIG_DIR = Path(__file__).resolve().parent
MISSING = "???"
_INTERP = re.compile(r"\$\{([^}]+)\}")


class ConfigError(ValueError):
    pass


class Config(dict):
    """dict with attribute access and dotted-path helpers."""

    def __getattr__(self, name: str) -> Any:
        try:
            return self[name]
        except KeyError as e:
            raise AttributeError(name) from e

    def __setattr__(self, name: str, value: Any) -> None:
        self[name] = value

    def get_path(self, path: str, default: Any = None) -> Any:
        node: Any = self
        for part in path.split("."):
            if not isinstance(node, dict) or part not in node:
                return default
            node = node[part]
        return node

    def set_path(self, path: str, value: Any, create: bool = True) -> None:
        node: Any = self
        parts = path.split(".")
        for part in parts[:-1]:
            if part not in node or not isinstance(node[part], dict):
                if not create:
                    raise ConfigError(f"no such config group: {path}")
                node[part] = Config()
            node = node[part]
        node[parts[-1]] = _wrap(value)

    def to_dict(self) -> dict:
        return _unwrap(self)


def _wrap(v: Any) -> Any:
    if isinstance(v, dict) and not isinstance(v, Config):
        return Config({k: _wrap(x) for k, x in v.items()})
    if isinstance(v, list):
        return [_wrap(x) for x in v]
    return v


def _unwrap(v: Any) -> Any:
    if isinstance(v, dict):
        return {k: _unwrap(x) for k, x in v.items()}
    if isinstance(v, list):
        return [_unwrap(x) for x in v]
    return v


def merge(base: dict, over: dict) -> dict:
    """Deep merge ``over`` into ``base`` (dicts merge, everything else replaces)."""
    for k, v in over.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            merge(base[k], v)
        else:
            base[k] = copy.deepcopy(v)
    return base


def _search(name: str, searchpath: list[Path]) -> Path:
    for d in searchpath:
        for cand in (d / f"{name}.yaml", d / name):
            if cand.is_file():
                return cand
    raise ConfigError(f"config '{name}' not found in {[str(p) for p in searchpath]}")


def _load_file(path: Path, searchpath: list[Path]) -> dict:
    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    defaults = raw.pop("defaults", [])
    raw.pop("hydra", None)
    out: dict = {}
    self_merged = False
    for d in defaults:
        if d == "_self_":
            merge(out, raw)
            self_merged = True
        elif isinstance(d, str):
            merge(out, _load_file(_search(d, [path.parent] + searchpath), searchpath))
        elif isinstance(d, dict):
            for group, name in d.items():
                merge(out, {group: _load_file(_search(f"{group}/{name}", [path.parent] + searchpath), searchpath)})
    if not self_merged:
        merge(out, raw)
    return out


def parse_value(text: str) -> Any:
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def _resolve(node: Any, root: Config, stack: tuple = ()) -> Any:
    if isinstance(node, dict):
        for k in list(node.keys()):
            node[k] = _resolve(node[k], root, stack)
        return node
    if isinstance(node, list):
        return [_resolve(x, root, stack) for x in node]
    if isinstance(node, str) and "${" in node:
        def sub(m: re.Match) -> str:
            key = m.group(1).strip()
            if key.startswith("oc.env:") or key.startswith("env:"):
                name, _, default = key.split(":", 1)[1].partition(",")
                return os.environ.get(name.strip(), default.strip())
            if key in stack:
                raise ConfigError(f"interpolation cycle at {key}")
            val = root.get_path(key, MISSING)
            if val == MISSING:
                raise ConfigError(f"interpolation of missing key '{key}'")
            val = _resolve(val, root, stack + (key,))
            return val if isinstance(val, str) else yaml.safe_dump(val, default_flow_style=True).strip().removesuffix("...").strip()
        whole = _INTERP.fullmatch(node)
        if whole:
            key = whole.group(1).strip()
            if not key.startswith(("oc.env:", "env:")):
                val = root.get_path(key, MISSING)
                if val == MISSING:
                    raise ConfigError(f"interpolation of missing key '{key}'")
                return _resolve(copy.deepcopy(val), root, stack + (key,))
        return parse_value(_INTERP.sub(sub, node))
    return node


def _missing(node: Any, prefix: str = "") -> list[str]:
    out = []
    if isinstance(node, dict):
        for k, v in node.items():
            out += _missing(v, f"{prefix}{k}.")
    elif node == MISSING:
        out.append(prefix[:-1])
    return out


def compose(name: str = "training", overrides: list[str] | None = None, searchpath: list[str | Path] | None = None,
            check_missing: bool = True) -> Config:
    """Compose ``<name>.yaml`` with its defaults, then apply overrides in order.

    ``+group=file`` merges ``<group>/<file>.yaml`` from the search path at the root (a model family's overlay, the
    upstream ``+qwen3_5=config``); ``+a.b=v`` adds a key; ``a.b=v`` sets one; ``~a.b`` deletes one.
    """
    paths = [Path(p) for p in (searchpath or [])] + [CONFIG_DIR, CONFIG_DIR.parent / "models"]
    cfg = Config(_wrap(_load_file(_search(name, paths), paths)))
    for ov in overrides or []:
        if ov.startswith("~"):
            parts = ov[1:].split(".")
            node = cfg
            for p in parts[:-1]:
                node = node.get(p, {})
            node.pop(parts[-1], None)
            continue
        if "=" not in ov:
            raise ConfigError(f"override '{ov}' is not key=value")
        key, _, val = ov.partition("=")
        add = key.startswith("+")
        key = key.lstrip("+")
        if add and "." not in key:
            try:
                overlay = _load_file(_search(f"{key}/{val}", paths), paths)
                merge(cfg, _wrap(overlay))
                continue
            except ConfigError:
                pass
        if not add and cfg.get_path(key, MISSING) == MISSING and cfg.get_path(key, None) is None and not _exists(cfg, key):
            raise ConfigError(f"override of unknown key '{key}' (use +{key}=... to add it)")
        cfg.set_path(key, parse_value(val))
    cfg = Config(_wrap(_resolve(cfg, cfg)))
    if check_missing:
        miss = _missing(cfg)
        if miss:
            raise ConfigError(f"missing required config values: {miss}")
    return cfg


def _exists(cfg: Config, path: str) -> bool:
    node: Any = cfg
    for part in path.split("."):
        if not isinstance(node, dict) or part not in node:
            return False
        node = node[part]
    return True


def load_class(path: str):
    module_path, _, name = path.rpartition(".")
    return getattr(importlib.import_module(module_path), name)
