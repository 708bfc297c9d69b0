"""Block drafter for batch-1 speculative decoding: a 2-layer full-attention decoder of the target's hidden size that
reads the target's residual stream.

Row ``j`` of a draft pass combines the target residual of a committed position with the embedding of the token that
FOLLOWS it, ``x_j = fc([norm_e(embed(tok_{j+1})) | norm_h(residual_j)])`` (the MTP recipe of upstream
``rollout/blackwell/mtp.py:191-234``), and mask rows appended after the last committed row draft further positions
in the same pass (the block drafting of upstream ``deploy/blackwell/nvfp4/draft/proposal.py``). The drafter shares the
target's embedding and ``lm_head``; drafts are the argmax of its logits.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .config import HybridConfig
from .hybrid import DecoderLayer, RMSNorm, linear_fp32


class BlockDrafter(nn.Module):
    def __init__(self, cfg: HybridConfig, mask_token_id: int = 0):
        super().__init__()
        self.config = cfg
        self.mask_token_id = mask_token_id
        h = cfg.hidden_size
        self.pre_fc_norm_embedding = RMSNorm(h, cfg.rms_eps)
        self.pre_fc_norm_hidden = RMSNorm(h, cfg.rms_eps)
        self.fc = nn.Linear(2 * h, h, bias=False)
        self.layers = nn.ModuleList([DecoderLayer(cfg, "full_attention") for _ in range(cfg.num_layers)])
        self.norm = RMSNorm(h, cfg.rms_eps)

    def init_weights(self, seed: int = 1) -> "BlockDrafter":
        gen = torch.Generator().manual_seed(seed)
        for _, p in self.named_parameters():
            with torch.no_grad():
                if p.dim() >= 2:
                    p.copy_((torch.randn(p.shape, generator=gen) * self.config.init_std).to(p.dtype))
                else:
                    p.zero_()
        return self

    def fc_input(self, next_embeds: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        return torch.cat([self.pre_fc_norm_embedding(next_embeds), self.pre_fc_norm_hidden(residual)], dim=-1)

    def project(self, next_embeds: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        return linear_fp32(self.fc_input(next_embeds, residual), self.fc.weight)
