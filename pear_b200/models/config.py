"""Model shape of the hybrid Gated-DeltaNet + gated-attention decoder.

The 27B shape is the one the upstream kernels hard-code (hidden 5120: ``pear/models/qwen3_5/rollout/blackwell/csrc/
ar_norm.cu:210``; 24 q / 4 kv heads of 256: ``deploy/blackwell/nvfp4/csrc/attention.cuh:10``; GDN 16 qk / 48 v heads
of 128, conv width 4: ``deploy/blackwell/nvfp4/csrc/gdn_t.cuh:9-11``; FFN 17408: ``draft/csrc/dk_layout.cuh:10``;
vocab 2 x 124160: ``rollout/blackwell/draft_gemm_table.json``; M-RoPE sections (11, 11, 10) over 64 rotary channels:
``deploy/blackwell/nvfp4/step.py:66-67``).
"""

from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field


@dataclass
class HybridConfig:
    vocab_size: int = 248320
    hidden_size: int = 5120
    num_layers: int = 64
    full_attention_interval: int = 4  # layers i with (i + 1) % interval == 0 are full attention, the rest GDN
    # gated full attention
    num_attention_heads: int = 24
    num_kv_heads: int = 4
    head_dim: int = 256
    rotary_dim: int = 64
    rope_theta: float = 10_000_000.0
    mrope_sections: tuple[int, int, int] = (11, 11, 10)
    # gated delta net
    gdn_qk_heads: int = 16
    gdn_v_heads: int = 48
    gdn_head_dim: int = 128
    conv_kernel: int = 4
    # mlp / norm
    intermediate_size: int = 17408
    rms_eps: float = 1e-6
    l2_eps: float = 1e-6
    # multi-token prediction head
    num_mtp_layers: int = 1
    attn_output_gate: bool = True  # q_proj yields [q | gate] per head; False: plain attention (drafter)
    init_std: float = 0.02
    layer_types: list[str] = field(default_factory=list)

    def __post_init__(self) -> None:
        self.mrope_sections = tuple(self.mrope_sections)
        if not self.layer_types:
            self.layer_types = [
                "full_attention" if (i + 1) % self.full_attention_interval == 0 else "linear_attention"
                for i in range(self.num_layers)
            ]
        if len(self.layer_types) != self.num_layers:
            raise ValueError(f"layer_types has {len(self.layer_types)} entries for {self.num_layers} layers")
        if self.num_attention_heads % self.num_kv_heads:
            raise ValueError("num_attention_heads must be a multiple of num_kv_heads")
        if self.gdn_v_heads % self.gdn_qk_heads:
            raise ValueError("gdn_v_heads must be a multiple of gdn_qk_heads")
        if sum(self.mrope_sections) * 2 != self.rotary_dim:
            raise ValueError("mrope_sections must sum to rotary_dim / 2")
        if self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim exceeds head_dim")

    # derived sizes -------------------------------------------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def gdn_key_dim(self) -> int:
        return self.gdn_qk_heads * self.gdn_head_dim

    @property
    def gdn_value_dim(self) -> int:
        return self.gdn_v_heads * self.gdn_head_dim

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_key_dim + self.gdn_value_dim

    @property
    def attention_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "full_attention"]

    @property
    def gdn_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "linear_attention"]

    def num_parameters(self, with_mtp: bool = False) -> int:
        h = self.hidden_size
        mlp = 3 * h * self.intermediate_size
        attn = h * ((2 if self.attn_output_gate else 1) * self.q_size) + 2 * h * self.kv_size + self.q_size * h + 2 * self.head_dim
        gdn = (
            h * self.gdn_conv_dim + h * self.gdn_value_dim + 2 * h * self.gdn_v_heads
            + self.gdn_conv_dim * self.conv_kernel + 2 * self.gdn_v_heads + self.gdn_head_dim + self.gdn_value_dim * h
        )
        total = 2 * self.vocab_size * h + h
        for t in self.layer_types:
            total += mlp + 2 * h + (attn if t == "full_attention" else gdn)
        if with_mtp:
            total += self.num_mtp_layers * (2 * h * h + 4 * h + attn + mlp + h)
        return total

    def flops_per_token(self, context: int = 0) -> float:
        """Forward matmul FLOPs per token (2 x weights touched) plus attention over ``context`` keys."""
        dense = 2.0 * (self.num_parameters() - self.vocab_size * self.hidden_size)
        attn = 4.0 * len(self.attention_layers) * self.num_attention_heads * self.head_dim * context
        gdn = 6.0 * len(self.gdn_layers) * self.gdn_v_heads * self.gdn_head_dim * self.gdn_head_dim
        return dense + attn + gdn

    # presets -------------------------------------------------------------------------------------------------------
    @classmethod
    def qwen3_8_27b(cls) -> "HybridConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "HybridConfig":
        """4 layers (3 GDN + 1 attention), hidden 256: the CPU plumbing configuration."""
        return cls(
            vocab_size=1024, hidden_size=256, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=64,
            rotary_dim=32, mrope_sections=(6, 5, 5), gdn_qk_heads=4, gdn_v_heads=4, gdn_head_dim=64,
            intermediate_size=768, num_mtp_layers=1,
        )

    @classmethod
    def small_gpu(cls) -> "HybridConfig":
        """A few layers of the 27B per-layer shape: kernels see their production tile sizes, memory stays small."""
        return cls(num_layers=4, vocab_size=32768)

    @classmethod
    def drafter(cls, hidden_size: int = 5120, vocab_size: int = 248320) -> "HybridConfig":
        """2-layer full-attention drafter of the target's hidden size (32 q / 8 kv heads of 128, FFN 17408), the
        shape of the upstream DFlash-2 draft (``deploy/blackwell/nvfp4/draft/csrc/dk_layout.cuh``)."""
        return cls(
            vocab_size=vocab_size, hidden_size=hidden_size, num_layers=2, full_attention_interval=1,
            num_attention_heads=32, num_kv_heads=8, head_dim=128, rotary_dim=64, intermediate_size=17408,
            num_mtp_layers=0, attn_output_gate=False,
        )

    # io ------------------------------------------------------------------------------------------------------------
    def to_dict(self) -> dict:
        d = dataclasses.asdict(self)
        d["mrope_sections"] = list(self.mrope_sections)
        d["model_type"] = "pear_hybrid"
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "HybridConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=1)

    @classmethod
    def load(cls, path: str) -> "HybridConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))
