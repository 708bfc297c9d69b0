"""Pictures of an observation -> the embedding rows that replace their image-pad tokens, on the agent-loop side.

Environments hand over either finished embedding blocks (``[tokens, hidden]`` floats: the seeded synthetic family) or pixels
(``[H, W, 3]`` uint8: a simulator's cameras). Pixels go through the vision tower here, once per distinct picture: a turn-based
episode shows the same frame again whenever the scene did not change, and every sample of a prompt group starts from the same
first frame, so encodings are kept in a small LRU keyed by the picture's bytes. The tower is shared by the agent-loop workers
(one batched call per observation, under a lock) and runs without gradients: the trainer receives the rows as part of the
trajectory, as it does for the synthetic family. (Upstream runs its tower inside the serving stack and again in the trainer:
pear/models/qwen3_5/trainer/vision_tower.py:11-133.)
"""

from __future__ import annotations

import hashlib
import threading
from collections import OrderedDict

import numpy as np
import torch


class VisionEncoder:
    def __init__(self, tower, device: str = "cpu", cache_entries: int = 512, pixel_dtype: torch.dtype = torch.float32,
                 min_pixels: int = 0, max_pixels: int = 1 << 22):
        """``min_pixels`` / ``max_pixels``: a camera picture whose sides are not multiples of the tower's patch x merge, or whose
        area is out of bounds, is resized first (the family's image-processor rule, ``eval/general.py: picture_size``)."""
        from ..models.vision import tower_cell

        self.cell = tower_cell(tower.cfg)
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.tower = tower.to(device).eval()
        self.device, self.pixel_dtype = torch.device(device), pixel_dtype
        self.cache: "OrderedDict[bytes, np.ndarray]" = OrderedDict()
        self.cache_entries = cache_entries
        self.lock = threading.Lock()
        self.encoded = self.hits = 0

    def follow(self, state: dict, version: int = 0, prefix: str = "visual.") -> None:
        """Take the tower's weights out of a trainer state (``WeightSync`` listener): encodings of the previous policy are dropped."""
        own = dict(self.tower.state_dict())
        mine = {k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix) and k[len(prefix):] in own}
        if not mine:
            return
        with self.lock:
            with torch.no_grad():
                for k, v in mine.items():
                    own[k].copy_(v.to(own[k].dtype))
            self.cache.clear()

    def grid(self, frame: np.ndarray) -> tuple[int, int]:
        """(rows, columns) of the block a pixel frame is encoded to."""
        from ..models.vision import picture_size

        h, w = picture_size(frame.shape[0], frame.shape[1], self.cell, self.min_pixels, self.max_pixels)
        return h // self.cell, w // self.cell

    @staticmethod
    def is_pixels(frame: np.ndarray) -> bool:
        return frame.ndim == 3 and frame.dtype == np.uint8

    def _prepare(self, frame: np.ndarray) -> torch.Tensor:
        """[H, W, C] uint8 -> [C, H, W] in [-1, 1]; ``pixel_dtype`` is the precision pixels are handed over in (the tower itself
        computes in fp32)."""
        from ..models.vision import prepare_picture

        return prepare_picture(np.ascontiguousarray(frame), self.cell, self.min_pixels, self.max_pixels, self.device, self.pixel_dtype)

    def encode(self, frames: list[np.ndarray]) -> list[np.ndarray]:
        out: list = [None] * len(frames)
        todo: list[tuple[int, bytes]] = []
        with self.lock:
            for i, f in enumerate(frames):
                if not self.is_pixels(f):
                    out[i] = np.asarray(f, dtype=np.float32)
                    continue
                key = hashlib.blake2b(f.tobytes(), digest_size=16, person=str(f.shape).encode()[:16]).digest()
                hit = self.cache.get(key)
                if hit is not None:
                    self.cache.move_to_end(key)
                    out[i] = hit
                    self.hits += 1
                else:
                    todo.append((i, key))
            if todo:
                first: dict[bytes, int] = {}
                for i, key in todo:  # the same picture twice in one observation is encoded once
                    first.setdefault(key, i)
                with torch.no_grad():
                    rows = self.tower([self._prepare(frames[i]) for i in first.values()])
                for key, block in zip(first, rows):
                    self.cache[key] = block.float().cpu().numpy()
                    self.encoded += 1
                while len(self.cache) > self.cache_entries:
                    self.cache.popitem(last=False)
                for i, key in todo:
                    out[i] = self.cache[key]
        return out


def build_vision_encoder(preset: str, model_path: str = "", hidden: int = 0, device: str = "cpu") -> "VisionEncoder":
    """The encoder a command-line option names: ``checkpoint`` (the family's tower with the model directory's sizes and
    ``model.visual.*`` tensors), ``family_<preset>`` (that architecture, random) or a preset of the small plain ViT (``tiny``);
    ``hidden`` is the decoder's width the rows are projected to (default: the model directory's)."""
    from ..models import io as model_io
    from ..models.vision import FamilyVisionConfig, FamilyVisionTower, VisionConfig, VisionTower

    if preset == "checkpoint":
        vcfg = model_io.load_vision_config(model_path)
        if vcfg is None:
            raise ValueError(f"{model_path} has no vision_config")
        tower = FamilyVisionTower(vcfg)
        own = dict(tower.state_dict())
        with torch.no_grad():
            for key, t in model_io.iter_model_tensors(model_path, only=lambda k: model_io.from_hf_name(k).startswith("visual.")):
                own[model_io.from_hf_name(key)[len("visual."):]].copy_(t.to(torch.float32))
    else:
        if not hidden:
            hidden = model_io.load_config(model_path).hidden_size if model_path and not model_path.startswith("preset:") else 256
        family = preset.startswith("family_")
        vcfg = getattr(FamilyVisionConfig if family else VisionConfig, preset[len("family_"):] if family else preset)(out_hidden=hidden)
        tower = (FamilyVisionTower if family else VisionTower)(vcfg).init_weights(0)
    return VisionEncoder(tower, device)
