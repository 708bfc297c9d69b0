"""A rollout replica that lives in another process, behind the HTTP app of :mod:`pear_b200.rollout.server`.

``RemoteReplica`` has the interface the agent-loop router and ``WeightSync`` use on an in-process ``RolloutServer``
(``generate``, ``pause``, ``resume``, ``release_cached_memory``, ``close``), so the trainer process can drive replicas that
were started as processes of their own (``python -m pear_b200.rollout.server``, the rollout role of ``launch/roles.py``) on
their own GPUs. Weights do not travel over HTTP: the replica process joins the trainer's weight-sync process group and
receives buckets through a ``weight_sync`` transport (``--sync-rank`` / ``--sync-world`` / ``--sync-master`` of the server
entry point). Upstream reaches its vLLM replicas the same way: HTTP for requests, a collective group for weights
(pear/rollout/async_server.py, pear/rollout/checkpoint_engine.py:15-43).
"""

from __future__ import annotations

import base64
import threading
import time
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .engine import FinishReason, SamplingParams


@dataclass
class RemoteRequest:
    """What a finished request looks like to the agent loop (the fields it reads of ``engine.Request``)."""

    request_id: str
    prompt: list
    output: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)
    topk_ids: list = field(default_factory=list)
    topk_logprobs: list = field(default_factory=list)
    finish: Optional[FinishReason] = None
    policy_version: int = 0
    cached_prefix: int = 0


def encode_embeds(embeds: Optional[torch.Tensor], mask: Optional[torch.Tensor]) -> dict:
    """Placeholder embedding rows of a prompt as JSON fields: bf16 bytes in base64 (the rows the mask selects only)."""
    if embeds is None:
        return {}
    m = mask.bool().cpu() if mask is not None else torch.ones(embeds.shape[0], dtype=torch.bool)
    rows = embeds.detach().cpu()[m].to(torch.bfloat16).contiguous()
    return {"embeds_b64": base64.b64encode(rows.view(torch.int16).numpy().tobytes()).decode("ascii"), "embeds_dim": int(embeds.shape[1]),
            "embeds_positions": torch.nonzero(m).flatten().tolist(), "embeds_len": int(embeds.shape[0])}


def decode_embeds(body: dict):
    """Inverse of :func:`encode_embeds`: (embeds [L, H] fp32 with zeros outside the mask, mask [L] bool) or (None, None)."""
    if "embeds_b64" not in body:
        return None, None
    dim, n, pos = int(body["embeds_dim"]), int(body["embeds_len"]), list(body["embeds_positions"])
    raw = np.frombuffer(base64.b64decode(body["embeds_b64"]), dtype=np.int16).copy()
    rows = torch.from_numpy(raw).view(torch.bfloat16).view(len(pos), dim).float()
    embeds, mask = torch.zeros(n, dim), torch.zeros(n, dtype=torch.bool)
    if pos:
        idx = torch.tensor(pos, dtype=torch.long)
        embeds[idx] = rows
        mask[idx] = True
    return embeds, mask


class RemoteReplica:
    def __init__(self, url: str, name: Optional[str] = None, timeout_s: float = 3600.0):
        import requests

        self.url, self.name, self.timeout_s = url.rstrip("/"), name or url, timeout_s
        self._local = threading.local()  # one HTTP session per calling thread
        self._requests = requests

    def _session(self):
        s = getattr(self._local, "session", None)
        if s is None:
            s = self._local.session = self._requests.Session()
        return s

    def _post(self, path: str, body: dict, timeout: Optional[float] = None) -> dict:
        r = self._session().post(self.url + path, json=body, timeout=timeout or self.timeout_s)
        r.raise_for_status()
        return r.json()

    def wait_ready(self, timeout_s: float = 300.0, alive=None) -> None:
        """Block until the replica answers ``/health``. ``alive``: a callable that tells whether the replica's process still
        runs (a launcher's ``lambda: proc.poll() is None``): a replica that died while starting is reported at once."""
        t0 = time.time()
        while True:
            if alive is not None and not alive():
                raise RuntimeError(f"{self.name}: the replica process ended before it answered on {self.url}/health")
            try:
                if self._session().get(self.url + "/health", timeout=5).json().get("ok"):
                    return
            except Exception:  # noqa: BLE001 - the process is still starting
                pass
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"{self.name}: no answer on {self.url}/health within {timeout_s} s")
            time.sleep(0.25)

    # -- the RolloutServer interface the router and WeightSync use ------------------------------------------------------
    def generate(self, prompt: list, params: Optional[SamplingParams] = None, session: Optional[str] = None, embeds=None, embeds_mask=None,
                 timeout_s: Optional[float] = None, max_resubmits: int = 1000, position_ids=None) -> RemoteRequest:
        p = params or SamplingParams()
        body = {"prompt_token_ids": list(map(int, prompt)), "max_tokens": p.max_tokens, "temperature": p.temperature, "top_p": p.top_p,
                "top_k": p.top_k, "seed": p.seed, "logprobs": p.topk_logprobs, "stop_token_ids": list(p.stop_token_ids), "session": session, "max_resubmits": max_resubmits}
        body.update(encode_embeds(embeds, embeds_mask))
        if position_ids is not None:
            body["position_ids"] = torch.as_tensor(position_ids).tolist()
        out = self._post("/v1/completions", body, timeout_s)
        if "error" in out:
            raise RuntimeError(f"{self.name}: {out['error']}")
        c = out["choices"][0]
        return RemoteRequest(out["id"], list(prompt), c["token_ids"], c["logprobs"], c.get("topk_ids") or [], c.get("topk_logprobs") or [],
                             FinishReason(c["finish_reason"]) if c.get("finish_reason") else None, int(out.get("policy_version", 0)),
                             int(out.get("cached_prefix", 0)))

    def pause(self, abort: bool = True) -> int:
        self._loads_at_pause = self._health().get("weight_loads", 0)  # a sync starts with a pause: wait_version counts from here
        return int(self._post("/pause", {"abort": abort}).get("aborted", 0))

    def resume(self) -> None:
        self._post("/resume", {})

    def release_cached_memory(self) -> None:
        self._post("/release_cached_memory", {})

    def metrics_text(self) -> str:
        return self._session().get(self.url + "/metrics", timeout=30).text

    def _health(self) -> dict:
        return self._session().get(self.url + "/health", timeout=30).json()

    def policy_version(self) -> int:
        return int(self._health().get("policy_version", 0))

    def wait_version(self, version: int, timeout_s: float = 600.0) -> None:
        """Block until the replica has loaded the weights of ``version`` (its receiver loads after the last bucket; requests
        released earlier would still be answered, and tagged, with the previous policy)."""
        t0, before = time.time(), getattr(self, "_loads_at_pause", -1)
        while True:
            h = self._health()
            if int(h.get("policy_version", 0)) == version and int(h.get("weight_loads", 0)) > before:
                return
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"{self.name} did not load policy version {version} within {timeout_s:.0f} s")
            time.sleep(0.02)

    def close(self) -> None:
        s = getattr(self._local, "session", None)
        if s is not None:
            s.close()
