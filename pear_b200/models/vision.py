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


def picture_size(height: int, width: int, multiple: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """The size a picture is resized to before the tower: both sides the nearest multiple of ``multiple`` (the tower's patch x
    merge), then scaled (aspect kept, sides floored / ceiled to multiples) so that the area lies in [min_pixels, max_pixels]: the
    rule of the family's image processor, checked against it in ``tests/test_hf_parity_cpu.py``."""
    import math

    h = max(multiple, round(height / multiple) * multiple)
    w = max(multiple, round(width / multiple) * multiple)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(multiple, math.floor(height / beta / multiple) * multiple)
        w = max(multiple, math.floor(width / beta / multiple) * multiple)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / multiple) * multiple
        w = math.ceil(width * beta / multiple) * multiple
    return h, w


def tower_cell(cfg) -> int:
    """Pixels per side of one output row's window: patch x merge of either tower's config."""
    return getattr(cfg, "patch_size", getattr(cfg, "patch", 1)) * getattr(cfg, "spatial_merge_size", getattr(cfg, "merge", 1))


def prepare_picture(frame, cell: int, min_pixels: int = 0, max_pixels: int = 1 << 22, device="cpu", pixel_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """uint8 ``[H, W, C]`` (array or tensor) -> ``[C, H', W']`` in [-1, 1] at :func:`picture_size`: what both the agent loop's
    encoder and the trainer feed a tower, so a picture gives the same rows on either side."""
    x = torch.as_tensor(frame).to(device).permute(2, 0, 1).to(pixel_dtype)
    x = (x / 127.5 - 1.0).float()
    h, w = picture_size(x.shape[1], x.shape[2], cell, min_pixels, max_pixels)
    if (h, w) != tuple(x.shape[1:]):
        x = F.interpolate(x[None], size=(h, w), mode="bicubic", align_corners=False, antialias=True)[0].clamp(-1.0, 1.0)
    return x


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


# ---------------------------------------------------------------------------------------------------------------------------
# The family's own tower (the `model.visual.*` tensors of its checkpoints)
# ---------------------------------------------------------------------------------------------------------------------------
@dataclass
class FamilyVisionConfig:
    """Sizes of the family's vision tower as its checkpoints' ``vision_config`` names them."""

    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    num_position_embeddings: int = 2304
    out_hidden_size: int = 3584
    rope_theta: float = 10000.0

    @classmethod
    def from_hf_dict(cls, d: dict) -> "FamilyVisionConfig":
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})

    @classmethod
    def tiny(cls, out_hidden: int = 256) -> "FamilyVisionConfig":
        return cls(depth=2, hidden_size=64, intermediate_size=128, num_heads=4, patch_size=4, num_position_embeddings=64, out_hidden_size=out_hidden)

    @property
    def out_hidden(self) -> int:
        return self.out_hidden_size


class _FamilyAttention(nn.Module):
    def __init__(self, cfg: FamilyVisionConfig):
        super().__init__()
        self.heads = cfg.num_heads
        self.qkv = nn.Linear(cfg.hidden_size, 3 * cfg.hidden_size)
        self.proj = nn.Linear(cfg.hidden_size, cfg.hidden_size)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """x [images, tokens, width] of one size; cos / sin [tokens, head_dim]: rotate-half rotary over (row, column)."""
        b, n, w = x.shape
        q, k, v = self.qkv(x).view(b, n, 3, self.heads, w // self.heads).permute(2, 0, 3, 1, 4)

        def rot(t):
            half = t.shape[-1] // 2
            return t * cos + torch.cat([-t[..., half:], t[..., :half]], dim=-1) * sin

        a = F.scaled_dot_product_attention(rot(q.float()), rot(k.float()), v.float())
        return self.proj(a.transpose(1, 2).reshape(b, n, w).to(x.dtype))


class _FamilyMLP(nn.Module):
    def __init__(self, cfg: FamilyVisionConfig):
        super().__init__()
        self.linear_fc1 = nn.Linear(cfg.hidden_size, cfg.intermediate_size)
        self.linear_fc2 = nn.Linear(cfg.intermediate_size, cfg.hidden_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear_fc2(F.gelu(self.linear_fc1(x), approximate="tanh"))


class _FamilyBlock(nn.Module):
    def __init__(self, cfg: FamilyVisionConfig):
        super().__init__()
        self.norm1 = nn.LayerNorm(cfg.hidden_size, eps=1e-6)
        self.norm2 = nn.LayerNorm(cfg.hidden_size, eps=1e-6)
        self.attn = _FamilyAttention(cfg)
        self.mlp = _FamilyMLP(cfg)

    def forward(self, x, cos, sin):
        x = x + self.attn(self.norm1(x), cos, sin)
        return x + self.mlp(self.norm2(x))


class _FamilyPatchEmbed(nn.Module):
    def __init__(self, cfg: FamilyVisionConfig):
        super().__init__()
        k = (cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size)
        self.proj = nn.Conv3d(cfg.in_channels, cfg.hidden_size, kernel_size=k, stride=k, bias=True)  # (kept as a convolution for its tensor names)


class _FamilyMerger(nn.Module):
    def __init__(self, cfg: FamilyVisionConfig):
        super().__init__()
        wide = cfg.hidden_size * cfg.spatial_merge_size ** 2
        self.norm = nn.LayerNorm(cfg.hidden_size, eps=1e-6)
        self.linear_fc1 = nn.Linear(wide, wide)
        self.linear_fc2 = nn.Linear(wide, cfg.out_hidden_size)


class FamilyVisionTower(nn.Module):
    """The vision tower of the model family's checkpoints (parameter names and arithmetic of ``model.visual.*``): a still picture
    is two identical frames under a temporal patch of two; patches are embedded by the (3-D) patch projection, a learned position
    table laid out on a square grid is interpolated bilinearly to the picture's patch grid and added; the blocks are pre-norm
    LayerNorm / full attention inside the picture with a rotate-half rotary embedding over (row, column) / tanh-GELU MLP; the
    merger normalises, concatenates every ``merge x merge`` window of patches and projects it to the language model's width.
    Tokens are kept in window-major order (all patches of a window are consecutive), which is the order the merger consumes.
    Same call interface as :class:`VisionTower`: ``tower(images)`` with ``[C, H, W]`` pictures gives one ``[tokens, out]`` block
    each. Checked against ``transformers``' implementation in ``tests/test_hf_parity_cpu.py``."""

    def __init__(self, cfg: FamilyVisionConfig):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = _FamilyPatchEmbed(cfg)
        self.pos_embed = nn.Embedding(cfg.num_position_embeddings, cfg.hidden_size)
        self.blocks = nn.ModuleList(_FamilyBlock(cfg) for _ in range(cfg.depth))
        self.merger = _FamilyMerger(cfg)
        self.side = int(cfg.num_position_embeddings ** 0.5)

    def init_weights(self, seed: int = 0) -> "FamilyVisionTower":
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)
                elif "norm" in name and name.endswith("weight"):
                    p.fill_(1.0)
                else:
                    p.zero_()
        return self

    def tokens_per_image(self, height: int, width: int) -> int:
        c = self.cfg
        return (height // c.patch_size // c.spatial_merge_size) * (width // c.patch_size // c.spatial_merge_size)

    def patches(self, img: torch.Tensor) -> tuple[torch.Tensor, int, int]:
        """[C, H, W] -> window-major patch vectors [gh * gw, C * Tp * P * P] (the checkpoint processor's ``pixel_values`` rows)."""
        c = self.cfg
        ch, h, w = img.shape
        p, m = c.patch_size, c.spatial_merge_size
        gh, gw = h // p, w // p
        if gh % m or gw % m or gh < m or gw < m:
            raise ValueError(f"picture {h}x{w}: the patch grid {gh}x{gw} must be a multiple of {m}")
        x = img[:, : gh * p, : gw * p].reshape(ch, gh // m, m, p, gw // m, m, p)
        x = x.permute(1, 4, 2, 5, 0, 3, 6)  # block row, block column, row in block, column in block, channel, y, x
        x = x.unsqueeze(5).expand(-1, -1, -1, -1, -1, c.temporal_patch_size, -1, -1)  # the still picture repeated over the temporal patch
        return x.reshape(gh * gw, ch * c.temporal_patch_size * p * p), gh, gw

    def _window_major(self, grid: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        m = self.cfg.spatial_merge_size
        return grid.reshape(gh // m, m, gw // m, m, -1).permute(0, 2, 1, 3, 4).reshape(gh * gw, -1)

    def _positions(self, gh: int, gw: int, device) -> torch.Tensor:
        """The position table interpolated bilinearly to a gh x gw grid, window-major: [gh * gw, width]."""
        s = self.side
        ys, xs = torch.linspace(0, s - 1, gh, device=device), torch.linspace(0, s - 1, gw, device=device)
        y0, x0 = ys.long(), xs.long()
        y1, x1 = (y0 + 1).clamp(max=s - 1), (x0 + 1).clamp(max=s - 1)
        fy, fx = (ys - y0)[:, None], (xs - x0)[None, :]
        table = self.pos_embed.weight

        def at(yy, xx):
            return table[(yy[:, None] * s + xx[None, :]).reshape(-1)].reshape(gh, gw, -1)

        out = (at(y0, x0) * ((1 - fy) * (1 - fx))[..., None] + at(y0, x1) * ((1 - fy) * fx)[..., None]
               + at(y1, x0) * (fy * (1 - fx))[..., None] + at(y1, x1) * (fy * fx)[..., None])
        return self._window_major(out, gh, gw)

    def _rotary(self, gh: int, gw: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        c = self.cfg
        hd = c.hidden_size // c.num_heads
        dim = hd // 2  # half of the head for rows, half for columns
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
        rows = torch.arange(gh, device=device, dtype=torch.float32)[:, None].expand(gh, gw)
        cols = torch.arange(gw, device=device, dtype=torch.float32)[None, :].expand(gh, gw)
        ang = torch.cat([rows[..., None] * inv, cols[..., None] * inv], dim=-1)  # [gh, gw, hd / 2]
        ang = self._window_major(ang, gh, gw)
        ang = torch.cat([ang, ang], dim=-1)  # [tokens, hd]
        return ang.cos(), ang.sin()

    def forward(self, images: list[torch.Tensor]) -> list[torch.Tensor]:
        c = self.cfg
        groups: dict[tuple[int, int], list[int]] = {}
        vecs = []
        for i, img in enumerate(images):
            v, gh, gw = self.patches(img.float())
            vecs.append(v)
            groups.setdefault((gh, gw), []).append(i)
        w = self.patch_embed.proj.weight.reshape(c.hidden_size, -1)
        out: list[torch.Tensor] = [None] * len(images)  # type: ignore[list-item]
        m2 = c.spatial_merge_size ** 2
        for (gh, gw), idx in groups.items():
            dev = vecs[idx[0]].device
            x = F.linear(torch.stack([vecs[i] for i in idx]), w, self.patch_embed.proj.bias) + self._positions(gh, gw, dev)
            cos, sin = self._rotary(gh, gw, dev)
            for blk in self.blocks:
                x = blk(x, cos, sin)
            x = self.merger.norm(x).reshape(len(idx), gh * gw // m2, m2 * c.hidden_size)
            y = self.merger.linear_fc2(F.gelu(self.merger.linear_fc1(x)))
            for j, i in enumerate(idx):
                out[i] = y[j]
        return out
