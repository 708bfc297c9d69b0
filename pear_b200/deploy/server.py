"""Deploy server: one checkpoint served to one session at a time (upstream ``pear/deploy/server/main.py:17-78``,
``worker_extension.py:8-19``): an OpenAI-style completion endpoint in front of the family's deploy engine (the batch-1
decode megakernel on a B200). Requests are serialised by a lock (``max_num_seqs 1``); the deploy kernels class is named
by class path in the recipe and exported through ``PEAR_DEPLOY_KERNELS``.

``MemoryPlan`` (upstream ``models/qwen3_5/deploy/memory_plan.py:22-182``) decides what stays in HBM: NVFP4 weights,
KV cache and GDN state for the configured context, and it moves the embedding table (and any vision tower) to pinned
host memory when the budget is short; rows are then fetched over PCIe/NVLink-C2C per token.
"""

from __future__ import annotations

import sys
import threading
import time
from dataclasses import dataclass
from typing import Optional

import torch

from ..config.loader import compose, load_class
from ..models.config import HybridConfig
from ..models.kernels import DeployKernels
from ..utils.tokenizer import ByteTokenizer


@dataclass
class MemoryPlan:
    weight_bytes: int
    kv_bytes: int
    state_bytes: int
    embedding_bytes: int
    embedding_on_host: bool
    total_device_bytes: int

    @classmethod
    def build(cls, cfg: HybridConfig, max_model_len: int, hbm_bytes: int = 180 << 30, utilization: float = 0.9,
              draft: Optional[HybridConfig] = None) -> "MemoryPlan":
        nvfp4 = lambda n: n // 2 + n // 16  # noqa: E731  codes + e4m3 block scales
        lin = cfg.num_parameters() - cfg.vocab_size * cfg.hidden_size  # everything but the embedding table
        weights = nvfp4(lin)
        if draft is not None:
            weights += nvfp4(draft.num_parameters() - 2 * draft.vocab_size * draft.hidden_size)
        kv = len(cfg.attention_layers) * 2 * max_model_len * cfg.kv_size * 2
        state = len(cfg.gdn_layers) * (cfg.gdn_v_heads * cfg.gdn_head_dim * cfg.gdn_head_dim * 4 + 3 * cfg.gdn_conv_dim * 4) * 2
        emb = cfg.vocab_size * cfg.hidden_size * 2
        budget = int(hbm_bytes * utilization)
        on_host = weights + kv + state + emb > budget
        total = weights + kv + state + (0 if on_host else emb)
        if total > budget:
            raise MemoryError(f"plan needs {total / 2**30:.1f} GiB of {budget / 2**30:.1f} GiB even with the embedding on the host: "
                              f"lower max_model_len ({max_model_len})")
        return cls(weights, kv, state, emb, on_host, total)


class DeployServer:
    def __init__(self, engine, tokenizer: Optional[ByteTokenizer] = None, name: str = "pear"):
        self.engine, self.tok, self.name = engine, tokenizer or ByteTokenizer(), name
        self.lock = threading.Lock()
        self.requests = 0
        self.tokens_out = 0
        self.busy_s = 0.0

    def complete(self, prompt_ids: list[int], max_tokens: int = 64, temperature: float = 1.0, seed: Optional[int] = None) -> dict:
        with self.lock:
            t0 = time.time()
            self.engine.temperature = float(temperature)
            if seed is not None:
                self.engine.seed = int(seed)
            res = self.engine.generate(torch.tensor(prompt_ids, dtype=torch.int32), max_tokens)
            dt = time.time() - t0
            self.requests += 1
            self.tokens_out += len(res.tokens)
            self.busy_s += dt
            return {"token_ids": list(res.tokens), "logprobs": list(getattr(res, "logprobs", [])), "seconds": dt,
                    "steps": getattr(res, "steps", None), "accepted_per_step": getattr(res, "accepted_per_step", None)}

    def metrics_text(self) -> str:
        return (f'pear_deploy_requests_total{{model="{self.name}"}} {self.requests}\n'
                f'pear_deploy_generation_tokens_total{{model="{self.name}"}} {self.tokens_out}\n'
                f'pear_deploy_busy_seconds_total{{model="{self.name}"}} {self.busy_s}\n')

    def generate(self, ids: list[int], params, session=None, embeds=None, embeds_mask=None):
        """The interface ``rollout/messages_api.py`` drives (a request object with ``output`` / ``finish`` / ``cached_prefix``): the
        deploy engine decodes a fixed number of tokens, so the answer is cut at the first stop token here."""
        from types import SimpleNamespace

        from ..rollout.engine import FinishReason

        if embeds is not None:
            raise ValueError("the deploy engine takes text prompts")
        toks = self.complete(list(ids), int(params.max_tokens), float(params.temperature), params.seed)["token_ids"]
        cut = next((i for i, t in enumerate(toks) if t in params.stop_token_ids), None)
        if cut is None:
            return SimpleNamespace(output=toks, finish=FinishReason.LENGTH, cached_prefix=0)
        return SimpleNamespace(output=toks[:cut + 1], finish=FinishReason.STOP, cached_prefix=0)

    def http_app(self):
        from fastapi import FastAPI
        from fastapi.responses import PlainTextResponse

        from ..rollout import messages_api

        app = FastAPI(title=f"pear_b200 deploy {self.name}")
        # GET /v1/models (with the context limit), POST /v1/messages and /v1/messages/count_tokens: what the agent harness
        # (deploy/harness) asks of its model server
        messages_api.register(app, self, self.tok, None, int(getattr(self.engine, "max_len", 0)) or None)

        @app.get("/health")
        def health() -> dict:
            return {"ok": True}

        @app.get("/metrics", response_class=PlainTextResponse)
        def metrics() -> str:
            return self.metrics_text()

        @app.post("/v1/completions")
        def completions(body: dict) -> dict:
            ids = body.get("prompt_token_ids") or self.tok.encode(body["prompt"])
            out = self.complete(list(ids), int(body.get("max_tokens", 64)), float(body.get("temperature", 1.0)), body.get("seed"))
            return {"model": self.name, "choices": [{"text": self.tok.decode(out["token_ids"]), **out, "finish_reason": "length"}],
                    "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out["token_ids"])}}

        return app


def main(argv=None) -> int:
    cfg = compose("server", list(sys.argv[1:] if argv is None else argv))
    if not cfg.kernels:
        raise SystemExit("server config names no deploy kernels (compose with +<family>=deploy)")
    kernels = DeployKernels.export(str(cfg.kernels))
    assert kernels is load_class(str(cfg.kernels))
    ecfg = dict(cfg.engine)
    ecfg.update({"num_speculative_tokens": int(dict(cfg.speculative).get("num_speculative_tokens", 0))})
    kernels.configure_server(ecfg, int(cfg.engine.max_num_seqs), int(ecfg.get("max_num_batched_tokens", 8192)))
    engine = kernels.build_engine(str(cfg.model), cfg.draft, ecfg)
    from ..utils.tokenizer import load_tokenizer

    server = DeployServer(engine, tokenizer=load_tokenizer(str(cfg.model)), name=str(cfg.server.served_model_name))
    import uvicorn
    uvicorn.run(server.http_app(), host=str(cfg.server.host), port=int(cfg.server.port), log_level="warning")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
