"""Vision tower: images -> rows of the language model's hidden size that replace the image-pad tokens.

The role of upstream's fp32 vision tower (``trainer/vision_tower.py:11-133``, ``trainer/vision_attention.py:6-64``: a ViT
whose linears run as 3-term bf16 splits and whose attention runs one call per run of equal-size images): patches are
embedded by a linear layer over flattened ``patch x patch x channels`` pixels, a learned 2-D position table is added,
``depth`` pre-norm blocks (LayerNorm, bidirectional attention within each image, GELU MLP) follow, and a merger
concatenates every ``merge x merge`` neighbourhood and projects it to the language model's width. Computation is fp32
(the tower is small and its output feeds the fp32 residual stream); images of one size are batched into one attention
call.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class VisionConfig:
    patch: int = 14
    channels: int = 3
    width: int = 1152
    depth: int = 4
    heads: int = 16
    mlp_ratio: float = 4.0
    merge: int = 2
    max_grid: int = 64          # position table covers max_grid x max_grid patches
    out_hidden: int = 5120

    @classmethod
    def tiny(cls, out_hidden: int = 256) -> "VisionConfig":
        return cls(patch=4, width=64, depth=2, heads=4, merge=2, max_grid=16, out_hidden=out_hidden)


class VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.heads = cfg.heads
        self.norm1 = nn.LayerNorm(cfg.width)
        self.qkv = nn.Linear(cfg.width, 3 * cfg.width)
        self.proj = nn.Linear(cfg.width, cfg.width)
        self.norm2 = nn.LayerNorm(cfg.width)
        hidden = int(cfg.width * cfg.mlp_ratio)
        self.fc1 = nn.Linear(cfg.width, hidden)
        self.fc2 = nn.Linear(hidden, cfg.width)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: [images, patches, width] (images of one size): attention never crosses an image."""
        b, n, w = x.shape
        qkv = self.qkv(self.norm1(x)).view(b, n, 3, self.heads, w // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
        x = x + self.proj(a.transpose(1, 2).reshape(b, n, w))
        return x + self.fc2(F.gelu(self.fc1(self.norm2(x))))


class VisionTower(nn.Module):
    def __init__(self, cfg: VisionConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = nn.Linear(cfg.patch * cfg.patch * cfg.channels, cfg.width)
        self.pos = nn.Parameter(torch.zeros(cfg.max_grid, cfg.max_grid, cfg.width))
        self.blocks = nn.ModuleList(VisionBlock(cfg) for _ in range(cfg.depth))
        self.norm = nn.LayerNorm(cfg.width)
        self.merger = nn.Sequential(nn.Linear(cfg.merge * cfg.merge * cfg.width, cfg.width), nn.GELU(), nn.Linear(cfg.width, cfg.out_hidden))

    def init_weights(self, seed: int = 0) -> "VisionTower":
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)
                elif "norm" in name and name.endswith("weight"):
                    p.fill_(1.0)
                else:
                    p.zero_()  # biases: nn.Linear draws them from the global generator otherwise
        return self

    def tokens_per_image(self, height: int, width: int) -> int:
        c = self.cfg
        return (height // c.patch // c.merge) * (width // c.patch // c.merge)

    def _patchify(self, img: torch.Tensor) -> tuple[torch.Tensor, int, int]:
        """img [C, H, W] -> [gh * gw, patch * patch * C]."""
        c = self.cfg
        ch, h, w = img.shape
        gh, gw = h // c.patch, w // c.patch
        if gh % c.merge or gw % c.merge or gh > c.max_grid or gw > c.max_grid:
            raise ValueError(f"image {h}x{w}: the patch grid {gh}x{gw} must be a multiple of {c.merge} and at most {c.max_grid}")
        p = img[:, : gh * c.patch, : gw * c.patch].reshape(ch, gh, c.patch, gw, c.patch).permute(1, 3, 2, 4, 0)
        return p.reshape(gh * gw, c.patch * c.patch * ch), gh, gw

    def forward(self, images: list[torch.Tensor]) -> list[torch.Tensor]:
        """One [tokens, out_hidden] fp32 block per image, in input order; equal-size images share the batched calls."""
        c = self.cfg
        groups: dict[tuple[int, int], list[int]] = {}
        patches = []
        for i, img in enumerate(images):
            p, gh, gw = self._patchify(img.float())
            patches.append(p)
            groups.setdefault((gh, gw), []).append(i)
        out: list[torch.Tensor] = [None] * len(images)  # type: ignore[list-item]
        for (gh, gw), idx in groups.items():
            x = self.patch_embed(torch.stack([patches[i] for i in idx])) + self.pos[:gh, :gw].reshape(1, gh * gw, c.width)
            for blk in self.blocks:
                x = blk(x)
            x = self.norm(x).view(len(idx), gh // c.merge, c.merge, gw // c.merge, c.merge, c.width)
            x = x.permute(0, 1, 3, 2, 4, 5).reshape(len(idx), (gh // c.merge) * (gw // c.merge), c.merge * c.merge * c.width)
            y = self.merger(x)
            for j, i in enumerate(idx):
                out[i] = y[j]
        return out
