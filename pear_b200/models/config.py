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
    def tiny_gpu(cls) -> "HybridConfig":
        """The plumbing configuration with the head sizes the rollout kernels are built for (attention 256, GDN 128): a CPU
        trainer can step it and a GPU replica runs it through the batched step, also sharded over two ranks."""
        return cls(
            vocab_size=4096, hidden_size=512, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=256,
            gdn_qk_heads=2, gdn_v_heads=4, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=1,
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

    # Hugging Face layout of the family's config.json: the decoder's fields sit under "text_config" with the transformers
    # names (num_hidden_layers, num_key_value_heads, linear_* for the Gated-DeltaNet mixer, partial_rotary_factor,
    # rope_parameters with the M-RoPE sections, mtp_num_hidden_layers).
    def to_hf_dict(self) -> dict:
        text = {
            "model_type": "qwen3_5_text", "vocab_size": self.vocab_size, "hidden_size": self.hidden_size, "num_hidden_layers": self.num_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_kv_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "rms_norm_eps": self.rms_eps, "hidden_act": "silu",
            "partial_rotary_factor": self.rotary_dim / self.head_dim, "full_attention_interval": self.full_attention_interval,
            "layer_types": list(self.layer_types), "attn_output_gate": self.attn_output_gate,
            "rope_parameters": {"rope_type": "default", "rope_theta": self.rope_theta, "mrope_interleaved": True,
                                "mrope_section": list(self.mrope_sections), "partial_rotary_factor": self.rotary_dim / self.head_dim},
            "linear_num_key_heads": self.gdn_qk_heads, "linear_num_value_heads": self.gdn_v_heads, "linear_key_head_dim": self.gdn_head_dim,
            "linear_value_head_dim": self.gdn_head_dim, "linear_conv_kernel_dim": self.conv_kernel, "mtp_num_hidden_layers": self.num_mtp_layers,
            "initializer_range": self.init_std, "l2_norm_eps": self.l2_eps, "dtype": "bfloat16", "tie_word_embeddings": False,
        }
        return {"architectures": ["Qwen3_5ForConditionalGeneration"], "model_type": "qwen3_5", "text_config": text, "tie_word_embeddings": False}

    @classmethod
    def from_hf_dict(cls, d: dict) -> "HybridConfig":
        t = d.get("text_config", d)
        need = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "vocab_size", "intermediate_size")
        lost = [k for k in need if k not in t]
        if lost:
            raise KeyError(f"config.json lacks {lost}: neither this framework's field names nor the Hugging Face text_config names were found")
        rope = t.get("rope_parameters") or t.get("rope_scaling") or {}
        head_dim = int(t.get("head_dim", t["hidden_size"] // t["num_attention_heads"]))
        factor = float(rope.get("partial_rotary_factor", t.get("partial_rotary_factor", 0.25)))
        rotary = int(round(head_dim * factor))
        sections = tuple(rope.get("mrope_section", ())) or None
        if sections is None or 2 * sum(sections) != rotary:
            half = rotary // 2
            sections = (half - 2 * (half // 3), half // 3, half // 3)
        kd, vd = int(t.get("linear_key_head_dim", 128)), int(t.get("linear_value_head_dim", 128))
        if kd != vd:
            raise ValueError("Gated-DeltaNet key and value head dimensions differ: not supported")
        kw = dict(
            vocab_size=int(t["vocab_size"]), hidden_size=int(t["hidden_size"]), num_layers=int(t["num_hidden_layers"]),
            num_attention_heads=int(t["num_attention_heads"]), num_kv_heads=int(t["num_key_value_heads"]), head_dim=head_dim, rotary_dim=rotary,
            rope_theta=float(rope.get("rope_theta", t.get("rope_theta", 10_000_000.0))), mrope_sections=sections,
            gdn_qk_heads=int(t.get("linear_num_key_heads", 16)), gdn_v_heads=int(t.get("linear_num_value_heads", 48)), gdn_head_dim=kd,
            conv_kernel=int(t.get("linear_conv_kernel_dim", 4)), intermediate_size=int(t["intermediate_size"]), rms_eps=float(t.get("rms_norm_eps", 1e-6)),
            l2_eps=float(t.get("l2_norm_eps", 1e-6)), num_mtp_layers=int(t.get("mtp_num_hidden_layers", 0)),
            attn_output_gate=bool(t.get("attn_output_gate", True)), init_std=float(t.get("initializer_range", 0.02)),
            full_attention_interval=int(t.get("full_attention_interval", 4)),
        )
        if t.get("layer_types"):
            kw["layer_types"] = list(t["layer_types"])
        return cls(**kw)

    def save(self, path: str, hf: bool = True, dtype: str = "bfloat16") -> None:
        """``hf``: the Hugging Face layout (loadable by transformers-style tools); this framework's own flat field names are
        added under "pear_b200" so nothing is lost in a round trip. ``dtype``: the element type of the tensors saved beside it
        (transformers loads a checkpoint in the type its config names)."""
        d = self.to_hf_dict() if hf else self.to_dict()
        if hf:
            d["pear_b200"] = self.to_dict()
            for section in (d, d.get("text_config", {})):
                if "dtype" in section:
                    section["dtype"] = dtype
        with open(path, "w") as f:
            json.dump(d, f, indent=1)

    @classmethod
    def load(cls, path: str) -> "HybridConfig":
        with open(path) as f:
            d = json.load(f)
        if "pear_b200" in d:
            return cls.from_dict(d["pear_b200"])
        if "text_config" in d or "num_hidden_layers" in d:
            return cls.from_hf_dict(d)
        if "num_layers" not in d:
            raise KeyError(f"{path}: not a model config of this framework nor a Hugging Face config (no num_layers / num_hidden_layers)")
        return cls.from_dict(d)
