"""Rollout replica server: one engine, one scheduling thread, thread-safe submission.

The role of upstream ``pear/rollout/server.py:14-82`` (a vLLM HTTP server subclass per replica) and of its worker
extension (``worker_extension.py:13-70``) without vLLM: requests are submitted from any thread and resolve to a
``Request`` when finished; ``pause(abort=True)`` ends in-flight requests as ABORTED at once (the caller resubmits them,
which is what upstream's patched pause does); ``update_weights`` refuses to run while requests are in flight, casts to
the rollout dtype except for the modules that must stay fp32, reloads in place and clears every KV tier
(``rollout/lmcache.py:263-274``); ``metrics_text()`` is the Prometheus exposition the monitor scrapes
(``monitor/metrics.py:88-97``); ``http_app()`` wraps the same calls as a small FastAPI application.
"""

from __future__ import annotations

import threading
import time
from concurrent.futures import Future
from typing import Iterable, Optional

import torch

from .engine import EngineConfig, FinishReason, Request, RolloutEngine, SamplingParams

PROM_COUNTERS = ("prompt_tokens", "generation_tokens", "preemptions", "aborted", "spec_drafted", "spec_accepted", "requests_finished",
                 "request_seconds", "first_tokens", "first_token_seconds",  # (the *_seconds sums over their counts give mean latencies)
                 "prefix_cache_queries", "prefix_cache_hits", "external_prefix_cache_hits")  # tokens looked up / found on the device / found in the host tier
PROM_GAUGES = ("num_running", "num_waiting", "policy_version", "free_blocks", "cached_blocks")


class RolloutServer:
    def __init__(self, engine: RolloutEngine, name: str = "replica-0", fp32_modules: Iterable[str] = (),
                 rollout_dtype: torch.dtype = torch.bfloat16, idle_sleep_s: float = 0.001):
        self.engine, self.name = engine, name
        self.fp32_modules = tuple(fp32_modules)
        self.rollout_dtype = rollout_dtype
        self.lock = threading.RLock()
        self.futures: dict[str, Future] = {}
        self.stop_flag = False
        self.idle_sleep_s = idle_sleep_s
        self.error: Optional[BaseException] = None
        self.sync_error: Optional[BaseException] = None  # set by the weight-sync receiver thread of a replica process
        self.weight_loads = 0
        self.thread = threading.Thread(target=self._loop, daemon=True, name=f"{name}-scheduler")
        self.thread.start()

    # -- scheduling thread --------------------------------------------------------------------------------------------
    def _resolve(self, reqs: Iterable[Request]) -> None:
        for r in reqs:
            f = self.futures.pop(r.request_id, None)
            if f is not None and not f.done():
                f.set_result(r)

    def _loop(self) -> None:
        # A new host thread starts on device 0: the kernel library launches on the thread's CURRENT device and stream, so a
        # replica on another GPU must select it here (torch's own ops switch devices per tensor and would hide the mistake:
        # the library's kernels would run on GPU 0 against the other GPU's memory).
        dev = next(self.engine.model.parameters()).device
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        while not self.stop_flag:
            try:
                with self.lock:
                    finished = self.engine.step() if (self.engine.has_work() and not self.engine.paused) else []
                    self._resolve(finished)
                    idle = not self.engine.has_work() or self.engine.paused
            except BaseException as e:  # noqa: BLE001 - surfaced to every waiter
                self.error = e
                with self.lock:
                    for f in self.futures.values():
                        if not f.done():
                            f.set_exception(e)
                    self.futures.clear()
                return
            if idle:
                time.sleep(self.idle_sleep_s)

    # -- client API ---------------------------------------------------------------------------------------------------
    def submit(self, prompt: list[int], params: Optional[SamplingParams] = None, session: Optional[str] = None,
               embeds=None, embeds_mask=None, position_ids=None) -> Future:
        if self.error is not None:
            raise RuntimeError(f"{self.name}: scheduler stopped") from self.error
        fut: Future = Future()
        with self.lock:
            req = self.engine.add_request(prompt, params, session, embeds=embeds, embeds_mask=embeds_mask, position_ids=position_ids)
            fut.request = req  # (a streaming caller reads the tokens produced so far while the future is pending)
            if req.finish is not None:  # rejected by a paused engine
                fut.set_result(req)
            else:
                self.futures[req.request_id] = fut
        return fut

    def generate(self, prompt: list[int], params: Optional[SamplingParams] = None, session: Optional[str] = None,
                 embeds=None, embeds_mask=None, timeout_s: Optional[float] = None, max_resubmits: int = 1000, position_ids=None) -> Request:
        """Blocking generate that resubmits a request the engine aborted for a weight sync (keeping what it produced)."""
        for _ in range(max_resubmits):
            req = self.submit(prompt, params, session, embeds, embeds_mask, position_ids).result(timeout=timeout_s)
            if req.finish != FinishReason.ABORTED:
                return req
            while self.engine.paused and not self.stop_flag:
                time.sleep(self.idle_sleep_s)
        raise RuntimeError(f"{self.name}: request aborted {max_resubmits} times")

    # -- control (weight sync) ----------------------------------------------------------------------------------------
    def pause(self, abort: bool = True) -> int:
        with self.lock:
            aborted = self.engine.pause(abort=abort)
            self._resolve(aborted)
        return len(aborted)

    def resume(self) -> None:
        with self.lock:
            self.engine.resume()

    def check_fp32_modules(self) -> list[str]:
        """Names of parameters that must be fp32 but are not (upstream ``worker_extension.py:38-70``)."""
        bad = []
        for name, p in self.engine.model.named_parameters():
            if any(m in name for m in self.fp32_modules) and p.dtype != torch.float32:
                bad.append(name)
        return bad

    def release_cached_memory(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def update_weights(self, state: dict[str, torch.Tensor], version: int) -> None:
        bad = self.check_fp32_modules()
        if bad:
            raise RuntimeError(f"{self.name}: modules that must stay fp32 are not: {bad[:4]}")
        cast = {}
        for name, t in state.items():
            keep32 = any(m in name for m in self.fp32_modules)
            cast[name] = t if (keep32 or not t.is_floating_point()) else t.to(self.rollout_dtype)
        with self.lock:
            self.engine.update_weights(cast, version)
            self.weight_loads += 1

    # -- observability ------------------------------------------------------------------------------------------------
    def stats(self) -> dict:
        with self.lock:
            return self.engine.stats()

    def metrics_text(self) -> str:
        s = self.stats()
        lines = []
        for k in PROM_COUNTERS:
            lines += [f"# TYPE pear_{k}_total counter", f'pear_{k}_total{{replica="{self.name}"}} {float(s.get(k, 0))}']
        for k in PROM_GAUGES:
            lines += [f"# TYPE pear_{k} gauge", f'pear_{k}{{replica="{self.name}"}} {float(s.get(k, 0))}']
        return "\n".join(lines) + "\n"

    def close(self) -> None:
        self.stop_flag = True
        self.thread.join(timeout=10)

    # -- HTTP ---------------------------------------------------------------------------------------------------------
    def http_app(self, tokenizer=None, vision=None, max_model_len: Optional[int] = None):
        """FastAPI application: POST /v1/completions (token ids or text), /v1/chat/completions, the Messages routes of
        ``messages_api.py`` (``vision``: the encoder of their image blocks), GET /metrics, POST /pause /resume."""
        from fastapi import FastAPI
        from fastapi.responses import PlainTextResponse

        app = FastAPI(title=f"pear_b200 rollout {self.name}")

        @app.get("/metrics", response_class=PlainTextResponse)
        def metrics() -> str:
            return self.metrics_text()

        @app.get("/health")
        def health() -> dict:
            return {"ok": self.error is None, "paused": self.engine.paused, "policy_version": self.engine.policy_version,
                    "weight_loads": self.weight_loads}

        @app.post("/v1/completions")
        def completions(body: dict) -> dict:
            prompt = body.get("prompt_token_ids")
            if prompt is None:
                if tokenizer is None:
                    return {"error": "text prompts need a tokenizer"}
                prompt = tokenizer.encode(body["prompt"])
            from .remote import decode_embeds

            params = SamplingParams(max_tokens=int(body.get("max_tokens", 64)), temperature=float(body.get("temperature", 1.0)),
                                    top_p=float(body.get("top_p", 1.0)), top_k=int(body.get("top_k", -1) or -1),
                                    seed=(int(body["seed"]) if body.get("seed") is not None else None), topk_logprobs=int(body.get("logprobs", 0) or 0),
                                    stop_token_ids=tuple(int(t) for t in body.get("stop_token_ids", ())))
            embeds, mask = decode_embeds(body)  # vision placeholder rows of a multi-modal prompt (bf16, base64)
            req = self.generate(list(prompt), params, session=body.get("session"), embeds=embeds, embeds_mask=mask,
                                max_resubmits=int(body.get("max_resubmits", 1000)), position_ids=body.get("position_ids"))
            out = {"id": req.request_id, "policy_version": req.policy_version, "cached_prefix": getattr(req, "cached_prefix", 0),
                   "choices": [{"token_ids": req.output, "logprobs": req.logprobs, "topk_ids": req.topk_ids, "topk_logprobs": req.topk_logprobs,
                                "finish_reason": req.finish.value if req.finish else None}],
                   "usage": {"prompt_tokens": len(req.prompt), "completion_tokens": len(req.output)}}
            if tokenizer is not None:
                out["choices"][0]["text"] = tokenizer.decode(req.output)
            return out

        @app.post("/v1/chat/completions")
        def chat(body: dict) -> dict:
            """The OpenAI chat form for third-party clients (benchmark harnesses, agent CLIs): ``messages`` are rendered with the
            tokenizer's chat template, the assistant header is opened, generation stops at the end-of-turn token."""
            if tokenizer is None:
                return {"error": "chat completions need a tokenizer"}
            ids: list[int] = []
            for m in body.get("messages", []):
                content = m.get("content", "")
                if isinstance(content, list):  # content parts: the text parts, in order
                    content = "".join(part.get("text", "") for part in content if part.get("type", "text") == "text")
                ids += tokenizer.render_turn(str(m.get("role", "user")), str(content))
            ids += tokenizer.generation_prompt()
            stops = (tokenizer.eos_id,) + tuple(getattr(tokenizer, "extra_stop_ids", ()))
            params = SamplingParams(max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or 256),
                                    temperature=float(body.get("temperature", 1.0)), top_p=float(body.get("top_p", 1.0)),
                                    top_k=int(body.get("top_k", -1) or -1), seed=(int(body["seed"]) if body.get("seed") is not None else None),
                                    stop_token_ids=stops)
            choices, completion_tokens = [], 0
            for i in range(int(body.get("n", 1))):
                req = self.generate(ids, params, session=body.get("user"))
                completion_tokens += len(req.output)
                text = tokenizer.decode([t for t in req.output if t not in stops], skip_special=True)
                choices.append({"index": i, "message": {"role": "assistant", "content": text},
                                "finish_reason": "stop" if req.finish == FinishReason.STOP else (req.finish.value if req.finish else None)})
            return {"id": f"chatcmpl-{req.request_id}", "object": "chat.completion", "model": body.get("model", self.name), "choices": choices,
                    "usage": {"prompt_tokens": len(ids), "completion_tokens": completion_tokens}}

        @app.post("/pause")
        def pause(body: Optional[dict] = None) -> dict:
            return {"aborted": self.pause(abort=bool((body or {}).get("abort", True)))}

        @app.post("/release_cached_memory")
        def release() -> dict:
            self.release_cached_memory()
            return {"ok": True}

        @app.post("/resume")
        def resume() -> dict:
            self.resume()
            return {"ok": True}

        from . import messages_api

        messages_api.register(app, self, tokenizer, vision, max_model_len)
        return app


def build_server(model, cfg: Optional[EngineConfig] = None, device="cpu", **kw) -> RolloutServer:
    return RolloutServer(RolloutEngine(model, cfg or EngineConfig(), device), **kw)


def apply_rollout_kernels(kernels_path: Optional[str], cfg: EngineConfig, model=None, tensor_parallel_size: int = 1) -> EngineConfig:
    """Run a model family's rollout hooks (``models/kernels.py: RolloutKernels``, named by ``rollout.kernels`` or exported in
    ``PEAR_ROLLOUT_KERNELS``) over a replica's engine settings: ``configure_server`` checks and completes them (KV page size,
    the batched-step switch, the batch limits), ``install_worker`` loads the kernel library before the model is used,
    ``check_model`` refuses another architecture. Returns the engine config to build with. (Upstream calls the same three
    hooks from its server and worker extension: pear/rollout/server.py:14-82, worker_extension.py:13-70.)"""
    import dataclasses
    import importlib

    from ..models.kernels import RolloutKernels

    if kernels_path:
        module_path, _, name = str(kernels_path).rpartition(".")
        kernels = getattr(importlib.import_module(module_path), name)
    else:
        kernels = RolloutKernels.from_env()
    if kernels is None:
        return cfg
    settings = {"block_size": cfg.block_size, "fast_decode": cfg.fast_decode, "tensor_parallel_size": tensor_parallel_size,
                "num_speculative_tokens": cfg.num_speculative_tokens}
    kernels.configure_server(settings, cfg.max_num_seqs, cfg.max_num_batched_tokens)
    kernels.install_worker(None)
    if model is not None:
        kernels.check_model(model, settings)
    known = {f.name for f in dataclasses.fields(cfg)}
    return dataclasses.replace(cfg, **{k: v for k, v in settings.items() if k in known})


def load_rollout_model(path: str, dtype: torch.dtype = torch.bfloat16, device: str = "cpu", with_mtp: bool = True, seed: int = 0,
                       drafter_path: Optional[str] = None):
    """``preset:<name>`` (random init of a ``HybridConfig`` preset) or a model directory in the Hugging Face layout.

    The MTP drafter of a model directory: trained checkpoints are exported without it, so it comes from ``drafter_path`` (the
    base model's directory; only its ``mtp.*`` tensors are read) and stays frozen across weight syncs; without
    ``drafter_path`` the directory's own ``mtp.*`` tensors are used when it has them, else the model comes up without a
    drafter (upstream: pear/rollout/server.py:22,32-35 loads the frozen drafter from files)."""
    from ..models import io as model_io
    from ..models.config import HybridConfig
    from ..models.hybrid import HybridForCausalLM

    if path.startswith("preset:"):
        cfg = getattr(HybridConfig, path.split(":", 1)[1])()
        model = HybridForCausalLM(cfg, with_mtp=with_mtp and cfg.num_mtp_layers > 0).init_weights(seed)
    else:
        cfg = model_io.load_config(path)
        source = drafter_path or path
        has_drafter = with_mtp and cfg.num_mtp_layers > 0 and any(model_io.from_hf_name(k).startswith("mtp.") for k in model_io.model_tensor_names(source))
        if drafter_path and with_mtp and not has_drafter:
            raise KeyError(f"{drafter_path} holds no mtp.* tensors")
        model = HybridForCausalLM(cfg, with_mtp=has_drafter)
        if has_drafter and drafter_path:
            model_io.load_model_dir(path, model, allow_missing=("mtp.",))  # everything but the drafter, strictly
            own = dict(model.state_dict())
            seen = set()
            with torch.no_grad():
                for key, t in model_io.iter_model_tensors(drafter_path, only=lambda k: model_io.from_hf_name(k).startswith("mtp.")):
                    name = model_io.from_hf_name(key)
                    if name in own:
                        if tuple(own[name].shape) != tuple(t.shape):
                            raise ValueError(f"{drafter_path}: tensor {key} has shape {tuple(t.shape)}, the drafter expects {tuple(own[name].shape)}")
                        own[name].copy_(t.to(own[name].dtype))
                        seen.add(name)
            lost = [k for k in own if k.startswith("mtp.") and k not in seen]
            if lost:
                raise KeyError(f"{drafter_path} lacks {len(lost)} drafter tensors (first: {lost[:4]})")
        else:
            model_io.load_model_dir(path, model, ignore_unexpected=("visual.",) if has_drafter else ("visual.", "mtp."))
    if device != "cpu":
        to_rollout_dtypes(model.to(device), dtype)
    return model.eval()


def to_rollout_dtypes(model, dtype: torch.dtype = torch.bfloat16):
    """The element types the rollout kernels read: matrices (embedding, projections, head) in ``dtype``; norm weights, the
    short conv, ``A_log`` and ``dt_bias`` stay fp32 (a model cast as a whole with ``.to(bfloat16)`` is refused by the kernel
    wrappers)."""
    for name, p in model.named_parameters():
        if p.dim() >= 2 and "conv1d" not in name:
            p.data = p.data.to(dtype)
    return model


def start_weight_receiver(server: RolloutServer, rank: int, world: int, master: str, src: int = 0, backend: str = "auto", device: str = "cpu",
                          heartbeat_s: float = 1.0, on_sender_gone=None):
    """Join the weight-sync process group ({sending trainer rank} + {replica ranks}) and load every sync the sender starts, on
    a thread of its own: each ``WeightSync.sync`` on the trainer side arrives here as buckets until the last one, then the
    replica loads them, bumps its policy version and clears its KV tiers. Returns the thread."""
    import threading

    import torch.distributed as dist

    from ..loop.weight_sync import BroadcastTransport, StandaloneGroup, SymmTransport, receive_all

    if backend == "auto":
        backend = "nccl" if device != "cpu" else "gloo"
    if backend == "nvswitch":  # symmetric memory rendezvous goes through the default world: this process has no other
        from ..parallel.symm import SymmWorld

        dist.init_process_group("nccl", init_method=f"tcp://{master}", rank=rank, world_size=world)
        transport = SymmTransport(SymmWorld(reductions=False), src, server.engine.model.config)
    else:  # a world of its own, beside a tensor-parallel world the replica may be part of
        group = StandaloneGroup(master, rank, world, backend, device)
        transport = BroadcastTransport(group, src, device if backend == "nccl" else "cpu")
        hb = group.heartbeat()
        server.leave_sync_world = lambda: hb.leave(server.weight_loads)  # a clean exit says so: the sender is told, not timed out

        def beat():
            while not server.stop_flag:
                try:
                    hb.beat(server.weight_loads)
                except Exception:  # noqa: BLE001 - the sender (and its store) is gone
                    return
                time.sleep(heartbeat_s)

        threading.Thread(target=beat, daemon=True, name=f"{server.name}-heartbeat").start()

    def loop():
        if device != "cpu":
            torch.cuda.set_device(next(server.engine.model.parameters()).device)  # a new thread starts on device 0
        while not server.stop_flag:
            try:
                receive_all(transport, server)
            except Exception as e:  # noqa: BLE001 - the group went away (the trainer exited): stop listening, keep serving
                if not server.stop_flag:
                    server.sync_error = e
                    if on_sender_gone is not None:
                        on_sender_gone()
                return

    t = threading.Thread(target=loop, daemon=True, name=f"{server.name}-weight-sync")
    t.start()
    return t


def main(argv=None) -> int:
    """``python -m pear_b200.rollout.server --model preset:tiny --port 8100``: one rollout replica as a process of its own
    (the rollout role of ``launch/roles.py``): builds the model and the engine on this process's GPU (CPU without one) and
    serves ``http_app`` until it is terminated. ``key=value`` arguments the launcher passes on to every role are ignored
    except ``actor_rollout_ref.model.path=`` and ``actor_rollout_ref.rollout.max_num_seqs=``."""
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8100)
    ap.add_argument("--name", default="replica-0")
    ap.add_argument("--num-blocks", type=int, default=2048)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--speculative-tokens", type=int, default=0)
    ap.add_argument("--host-gb", type=float, default=0.0, help="host-DRAM tier of the KV / state cache in GiB (also: actor_rollout_ref.rollout.custom.lmcache.enable=true and .l1_size_gb=...)")
    ap.add_argument("--numa", default="auto", help="NUMA node to run on and allocate the host tier from: auto (the GPU's node), none, or a number")
    ap.add_argument("--drafter", default=None, help="directory whose mtp.* tensors are the (frozen) drafter of a model directory without one")
    ap.add_argument("--vision", default="", help="vision encoder of the Messages routes' image blocks: checkpoint (the --model directory's tower), family_tiny, tiny")
    ap.add_argument("--check", action="store_true", help="build the replica, answer one request and exit (no HTTP server)")
    ap.add_argument("--sync-rank", type=int, default=-1, help="this replica's rank in the weight-sync process group (-1: no group)")
    ap.add_argument("--sync-world", type=int, default=0, help="size of the weight-sync group: the sending trainer rank + the replica ranks")
    ap.add_argument("--sync-master", default="127.0.0.1:29650", help="host:port of the weight-sync group's rendezvous")
    ap.add_argument("--sync-src", type=int, default=0, help="rank of the sender in the weight-sync group")
    ap.add_argument("--exit-with-trainer", action="store_true", help="leave (orderly) when the weight-sync world's sender is gone")
    ap.add_argument("--sync-backend", default="auto", choices=["auto", "gloo", "nccl", "nvswitch"],
                    help="nvswitch: pull this replica's shard out of the sender's symmetric staging buffer; gloo / nccl: broadcast")
    args, overrides = ap.parse_known_args(argv)
    from ..utils.process import die_with_parent, dump_stacks_on_signal
    from ..utils.tokenizer import load_tokenizer

    die_with_parent()
    dump_stacks_on_signal()
    kv = dict(o.split("=", 1) for o in overrides if "=" in o and not o.startswith("-"))
    path = args.model or kv.get("actor_rollout_ref.model.path", "preset:tiny")
    max_seqs = int(kv.get("actor_rollout_ref.rollout.max_num_seqs", args.max_num_seqs))
    # modules that stay fp32 in the replica (checked before every sync): the recipe's list, or the exported variable
    import os

    import yaml

    fp32_modules = tuple(yaml.safe_load(kv.get("actor_rollout_ref.rollout.fp32_modules", "null")) or
                         [m for m in os.environ.get("PEAR_ROLLOUT_FP32_MODULES", "").split(",") if m])
    device = "cuda" if torch.cuda.is_available() else "cpu"
    host_gb = args.host_gb
    if not host_gb and str(kv.get("actor_rollout_ref.rollout.custom.lmcache.enable", "false")).lower() == "true":
        host_gb = float(kv.get("actor_rollout_ref.rollout.custom.lmcache.l1_size_gb", 700))
    # bind to the GPU's NUMA node before anything large is allocated: the pinned host tier is touched by this process, and a
    # tier on the far socket halves the copy bandwidth of every store and load
    node = None
    if args.numa != "none":
        from ..utils.process import gpu_numa_node, set_numa_affinity, visible_gpu_index

        local = int(os.environ.get("LOCAL_RANK", "0"))
        node = int(args.numa) if args.numa != "auto" else (gpu_numa_node(visible_gpu_index(local)) if device == "cuda" else None)
        if node is not None and not set_numa_affinity(node):
            node = None
    ecfg = EngineConfig(num_blocks=args.num_blocks, max_num_seqs=max_seqs, num_speculative_tokens=args.speculative_tokens,
                        host_bytes=int(host_gb * (1 << 30)), host_numa_node=node)
    tp_rank, tp_world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    ecfg = apply_rollout_kernels(kv.get("actor_rollout_ref.rollout.kernels"), ecfg, tensor_parallel_size=tp_world)
    if tp_world > 1:  # one rank of a tensor-parallel replica (started under torch.distributed.run): lock-step with its peers
        import torch.distributed as dist

        from .lockstep import build_tp_replica

        if device == "cuda":  # the rank's GPU is chosen before the group exists and the group is bound to it
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
        server = build_tp_replica(path, ecfg, name=args.name, fp32_modules=fp32_modules)
        device = str(server.engine.device)
        if args.sync_backend == "nvswitch":
            raise SystemExit("--sync-backend nvswitch needs the default process group, which a tensor-parallel replica uses for its own ranks: use nccl")
    else:
        model = load_rollout_model(path, device=device, drafter_path=args.drafter)
        server = build_server(model, ecfg, device=device, name=args.name, fp32_modules=fp32_modules)
    if args.sync_rank >= 0:  # a tensor-parallel replica's ranks are consecutive in the weight-sync world
        gone = None
        if args.exit_with_trainer:  # a replica on a node of its own has nobody to stop it: it ends the way a launcher would end it
            import signal

            gone = lambda: os.kill(os.getpid(), signal.SIGTERM)  # noqa: E731
        start_weight_receiver(server, args.sync_rank + tp_rank, args.sync_world, args.sync_master, args.sync_src, args.sync_backend, device,
                              on_sender_gone=gone)
    try:
        if tp_world > 1 and tp_rank != 0:  # followers mirror the leader until its stop message
            import signal

            # the launcher signals every rank; a follower leaves only through the leader's stop message, between steps, so that
            # no rank ever waits on a peer that is gone
            signal.signal(signal.SIGTERM, lambda *_: None)
            while server.thread.is_alive():
                server.thread.join(0.5)
            return 0 if server.error is None else 1
        if args.check:
            r = server.generate(list(range(1, 20)), SamplingParams(max_tokens=4, temperature=1.0))
            print(f"{args.name}: {len(r.output)} tokens on {device}, finish {r.finish.value}")
            return 0
        import signal

        import uvicorn

        # uvicorn shuts down on SIGTERM / SIGINT and then raises the signal again under the handler it found: with the default
        # handler the process would end inside `run`, before a tensor-parallel leader has told its followers to stop
        signal.signal(signal.SIGTERM, lambda *_: None)
        signal.signal(signal.SIGINT, lambda *_: None)
        # a request that can no longer finish (a peer rank is gone) must not keep a terminated replica alive
        vision = None
        if args.vision:
            from ..loop.vision_encoder import build_vision_encoder

            vision = build_vision_encoder(args.vision, path, hidden=server.engine.runner.cfg.hidden_size, device=str(device))
        uvicorn.run(server.http_app(load_tokenizer(path), vision=vision), host=args.host, port=args.port, log_level="warning", timeout_graceful_shutdown=3)
        return 0
    finally:
        leave = getattr(server, "leave_sync_world", None)
        if leave is not None:
            try:
                leave()
            except Exception:  # noqa: BLE001 - the sender's store is gone already
                pass
        server.close()
        eng = server.engine
        print(f"{args.name} rank {tp_rank}: steps={eng.metrics['steps']} fast_steps={eng.fast.steps if eng.fast is not None else 0} "
              f"policy_version={eng.policy_version} weight_loads={server.weight_loads}", flush=True)
        if tp_world > 1:
            import torch.distributed as dist

            if device != "cpu":
                torch.cuda.synchronize()
            dist.destroy_process_group()


if __name__ == "__main__":
    raise SystemExit(main())
