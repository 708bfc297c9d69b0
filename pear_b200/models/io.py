"""Model directory I/O in the Hugging Face layout: ``config.json`` + ``model.safetensors`` (or shards with
``model.safetensors.index.json``).

The safetensors container is read and written here directly (8-byte little-endian header length, JSON header with
dtype / shape / data offsets, raw little-endian tensor bytes), so import / export need no extra dependency; files are
memory-mapped and tensors are views of the map until converted. Export writes fp32 for the modules that must stay
fp32 in the rollout and bf16 for the rest, and leaves the MTP head out on request (upstream ``model_merger.py:11-38``
exports without it; the drafter always comes from the base model).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Callable, Iterable, Iterator, Optional

import torch

from .config import HybridConfig

_DT = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
       "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
       "F8_E4M3": getattr(torch, "float8_e4m3fn", torch.uint8)}
_DT_REV = {v: k for k, v in _DT.items()}


def save_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: Optional[dict[str, str]] = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _DT_REV[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((-len(blob)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


class SafetensorsFile:
    """Lazy reader: ``keys()``, ``get(name)`` (a tensor copied out of the memory map)."""

    def __init__(self, path: str):
        self.path = path
        self.f = open(path, "rb")
        (n,) = struct.unpack("<Q", self.f.read(8))
        self.header = json.loads(self.f.read(n))
        self.metadata = self.header.pop("__metadata__", {})
        self.base = 8 + n
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> list[str]:
        return list(self.header)

    def get(self, name: str) -> torch.Tensor:
        h = self.header[name]
        lo, hi = h["data_offsets"]
        dt = _DT[h["dtype"]]
        if hi == lo:
            return torch.empty(h["shape"], dtype=dt)
        with warnings.catch_warnings():  # the map is read-only and the view is cloned before anyone could write
            warnings.simplefilter("ignore", UserWarning)
            buf = torch.frombuffer(self.mm, dtype=torch.uint8, count=hi - lo, offset=self.base + lo)
        return buf.view(dt).reshape(h["shape"]).clone()

    def close(self) -> None:
        self.mm.close()
        self.f.close()


def load_safetensors(path: str) -> dict[str, torch.Tensor]:
    f = SafetensorsFile(path)
    try:
        return {k: f.get(k) for k in f.keys()}
    finally:
        f.close()


def _model_files(directory: str) -> list[str]:
    index = os.path.join(directory, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as fh:
            return sorted(set(json.load(fh)["weight_map"].values()))
    return ["model.safetensors"]


def model_tensor_names(directory: str) -> list[str]:
    """The tensor names of a model directory, from the files' headers only (no tensor is read)."""
    names: list[str] = []
    for fn in _model_files(directory):
        f = SafetensorsFile(os.path.join(directory, fn))
        try:
            names += f.keys()
        finally:
            f.close()
    return names


def iter_model_tensors(directory: str, only: Optional[Callable[[str], bool]] = None) -> Iterator[tuple[str, torch.Tensor]]:
    """Stream (name, tensor) from a model directory, shard by shard (a 27B model never sits in host memory twice); ``only``
    selects by name before a tensor is read."""
    for fn in _model_files(directory):
        f = SafetensorsFile(os.path.join(directory, fn))
        try:
            for k in f.keys():
                if only is None or only(k):
                    yield k, f.get(k)
        finally:
            f.close()


HF_TEXT_PREFIX = "model.language_model."  # the decoder of the family's Hugging Face checkpoints (the reference model is
#                                            model.model.language_model.layers; its vision tower is model.visual.*, the drafter mtp.*)


def to_hf_name(name: str) -> str:
    """This framework's parameter name -> the Hugging Face checkpoint key."""
    if name.startswith("model.") and not name.startswith(HF_TEXT_PREFIX) and not name.startswith("model.visual."):
        return HF_TEXT_PREFIX + name[len("model."):]
    if name.startswith("visual."):
        return "model." + name
    return name  # lm_head.weight, mtp.*


def from_hf_name(key: str) -> str:
    """A Hugging Face checkpoint key (or already one of this framework's names) -> this framework's parameter name."""
    if key.startswith(HF_TEXT_PREFIX):
        return "model." + key[len(HF_TEXT_PREFIX):]
    if key.startswith("model.visual."):
        return key[len("model."):]
    return key


def save_model_dir(directory: str, config: HybridConfig, state: dict[str, torch.Tensor], fp32_modules: Iterable[str] = (),
                   dtype: torch.dtype = torch.bfloat16, drop_mtp: bool = True, max_shard_bytes: int = 4 << 30, hf_names: bool = True) -> list[str]:
    """Write a model directory: tensors under the Hugging Face key names (``hf_names``) and a Hugging Face config.json."""
    os.makedirs(directory, exist_ok=True)
    fp32_modules = tuple(fp32_modules)
    out: dict[str, torch.Tensor] = {}
    for name, t in state.items():
        if drop_mtp and name.startswith("mtp."):
            continue
        keep32 = any(m in name for m in fp32_modules)
        key = to_hf_name(name) if hf_names else name
        out[key] = t.detach().to(torch.float32 if keep32 else dtype) if t.is_floating_point() else t.detach()
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name in sorted(out):
        n = out[name].numel() * out[name].element_size()
        if size + n > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][name] = out[name]
        size += n
    files = []
    if len(shards) == 1:
        save_safetensors(os.path.join(directory, "model.safetensors"), shards[0], {"format": "pt"})
        files.append("model.safetensors")
    else:
        weight_map = {}
        for i, sh in enumerate(shards):
            fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_safetensors(os.path.join(directory, fn), sh, {"format": "pt"})
            files.append(fn)
            weight_map.update({k: fn for k in sh})
        with open(os.path.join(directory, "model.safetensors.index.json"), "w") as fh:
            json.dump({"metadata": {"total_size": sum(t.numel() * t.element_size() for t in out.values())}, "weight_map": weight_map}, fh)
    config.save(os.path.join(directory, "config.json"), hf=hf_names, dtype=str(dtype).replace("torch.", ""))
    return files


def load_model_dir(directory: str, model: torch.nn.Module, strict: bool = True, allow_missing: Iterable[str] = (),
                   ignore_unexpected: Iterable[str] = ("visual.", "mtp.")) -> tuple[list[str], list[str]]:
    """Copy a model directory's tensors into ``model`` in place; keys may be Hugging Face names or this framework's own.
    Returns (missing, unexpected) names. With ``strict`` (the default) a parameter of the model that the directory does not
    provide raises unless its name starts with one of ``allow_missing``, and so does a tensor of the directory the model has
    no place for unless it starts with one of ``ignore_unexpected`` (a text-only model reading a checkpoint that also
    carries the vision tower or the drafter): a model must never come up partly random without anybody noticing. A shape
    mismatch always raises."""
    own = dict(model.state_dict())
    seen = set()
    unexpected = []
    with torch.no_grad():
        for key, t in iter_model_tensors(directory):
            name = from_hf_name(key)
            if name in own:
                if tuple(own[name].shape) != tuple(t.shape):
                    raise ValueError(f"{directory}: tensor {key} has shape {tuple(t.shape)}, the model expects {tuple(own[name].shape)}")
                own[name].copy_(t.to(own[name].dtype))
                seen.add(name)
            else:
                unexpected.append(name)
    missing = [k for k in own if k not in seen]
    if strict:
        allow_missing, ignore_unexpected = tuple(allow_missing), tuple(ignore_unexpected)
        bad_missing = [k for k in missing if not k.startswith(allow_missing)] if allow_missing else missing
        bad_unexpected = [k for k in unexpected if not k.startswith(ignore_unexpected)] if ignore_unexpected else unexpected
        if bad_missing or bad_unexpected:
            raise KeyError(f"{directory} does not match the model: {len(bad_missing)} parameters missing (first: {bad_missing[:4]}), "
                           f"{len(bad_unexpected)} tensors unexpected (first: {bad_unexpected[:4]})")
    return missing, unexpected


def load_vision_config(directory: str):
    """The ``vision_config`` of a model directory's config.json as a ``FamilyVisionConfig`` (None: a text-only checkpoint)."""
    from .vision import FamilyVisionConfig

    with open(os.path.join(directory, "config.json")) as f:
        d = json.load(f)
    v = d.get("vision_config")
    return FamilyVisionConfig.from_hf_dict(v) if isinstance(v, dict) else None


def load_config(directory: str) -> HybridConfig:
    return HybridConfig.load(os.path.join(directory, "config.json"))
