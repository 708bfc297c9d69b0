"""General-capability evaluation, one protocol for every model compared (upstream ``pear/eval/general.py:16-353`` with the
protocol of ``pear/configs/general.yaml``; upstream runs the benchmarks as evalscope tasks against vLLM's OpenAI endpoint,
this build owns the runner and the scorers, ``eval/scorers.py``).

``python -m pear_b200.eval.general <command>``:

* ``run``: every benchmark of ``config/general.yaml`` (or ``--only``) against rollout replicas (``--replicas url,url`` of
  ``rollout/server.py`` processes, or ``--model`` for in-process replicas), all benchmarks in flight at once under one
  concurrency limit so the replicas see a steady stream instead of each benchmark's tail. Every finished sample is appended to
  ``OUT/<benchmark>/samples.jsonl``; a rerun on the same OUT reuses the finished samples when the benchmark's identity (its
  definition + the sampling protocol + the model name) is unchanged and sets them aside when it changed. One benchmark's
  failure does not stop the others; the command fails at the end naming them.
* ``datasets``: which benchmark files are present under ``--dataset-dir`` and how many items each holds (there is no network in
  this build's environment: files are fetched elsewhere; the config names each benchmark's source).
* ``router``: an HTTP proxy that sends each request to the replica with the fewest requests in flight.
* ``compare``: per benchmark each run's mean score with its standard error, and a paired bootstrap of the difference over the
  samples both runs finished (resamples, seed and confidence from the config), marked when the interval excludes 0.

A benchmark file is JSONL: ``{"id", "prompt", "answer" | "instructions" | "tests", ...}``; its ``kind`` selects the scorer.
"""

from __future__ import annotations

import hashlib
import json
import os
import random
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..rollout.engine import FinishReason, SamplingParams
from ..utils.files import atomic_write
from ..models.vision import picture_size  # noqa: F401  (re-exported: the rule lives beside the towers)
from . import scorers


class LeastInFlightRouter:
    def __init__(self, servers: list):
        self.servers, self.inflight, self.lock = servers, [0] * len(servers), threading.Lock()

    def generate(self, prompt: list[int], params: SamplingParams, embeds=None, embeds_mask=None):
        with self.lock:
            i = min(range(len(self.servers)), key=lambda j: self.inflight[j])
            self.inflight[i] += 1
        try:
            if embeds is None:
                return self.servers[i].generate(prompt, params)
            return self.servers[i].generate(prompt, params, embeds=embeds, embeds_mask=embeds_mask)
        finally:
            with self.lock:
                self.inflight[i] -= 1


@dataclass
class Item:
    id: str
    prompt: str
    answer: str = ""
    extra: dict = field(default_factory=dict)  # the item's other fields (instructions, tests, num_options, ...)

    def as_dict(self) -> dict:
        return {"id": self.id, "prompt": self.prompt, "answer": self.answer, **self.extra}


def load_benchmark(path: str, limit: Optional[int] = None) -> list[Item]:
    items = []
    with open(path) as f:
        for d in map(json.loads, filter(str.strip, f)):
            items.append(Item(str(d["id"]), d["prompt"], str(d.get("answer", "")), {k: v for k, v in d.items() if k not in ("id", "prompt", "answer")}))
            if limit is not None and len(items) >= limit:
                break
    return items


def exact_last_line(completion: str, answer: str) -> float:
    return scorers.exact_last_line(completion, {"answer": answer})


def run_benchmark(router: LeastInFlightRouter, tokenizer, items: list[Item], n: int = 1, temperature: float = 1.0, top_p: float = 0.95,
                  max_tokens: int = 256, scorer: Callable[[str, str], float] = exact_last_line, workers: int = 16) -> dict[str, list[float]]:
    """The small form: every item ``n`` times, scores by item id (no files)."""
    params = SamplingParams(max_tokens=max_tokens, temperature=temperature, top_p=top_p, stop_token_ids=(tokenizer.eos_id,))

    def one(item: Item) -> tuple[str, list[float]]:
        prompt = tokenizer.render_turn("user", item.prompt) + tokenizer.generation_prompt()
        out = []
        for _ in range(n):
            req = router.generate(prompt, params)
            out.append(scorer(tokenizer.decode([t for t in req.output if t != tokenizer.eos_id], skip_special=True), item.answer))
        return item.id, out

    with ThreadPoolExecutor(max_workers=workers) as ex:
        return dict(ex.map(one, items))


# -- the protocol -------------------------------------------------------------------------------------------------------------
def identity(benchmark: dict, sampling: dict, model_name: str) -> str:
    """What a finished sample depends on: a change of any of it invalidates the samples already on disk."""
    blob = json.dumps({"benchmark": {k: benchmark[k] for k in sorted(benchmark) if k != "source"}, "sampling": sampling, "model": model_name}, sort_keys=True)
    return hashlib.sha256(blob.encode()).hexdigest()[:16]


class SampleStore:
    """``OUT/<benchmark>/samples.jsonl`` (one line per finished (item, repeat)) beside ``identity.json``."""

    def __init__(self, out_dir: str, name: str, ident: str):
        self.dir = os.path.join(out_dir, name)
        os.makedirs(self.dir, exist_ok=True)
        self.path = os.path.join(self.dir, "samples.jsonl")
        id_path = os.path.join(self.dir, "identity.json")
        old = None
        if os.path.exists(id_path):
            with open(id_path) as f:
                old = json.load(f).get("identity")
        if old != ident and os.path.exists(self.path):  # another protocol's samples: set aside, never mixed in
            os.replace(self.path, os.path.join(self.dir, f"samples.{old or 'unknown'}.stale.jsonl"))
        atomic_write(id_path, json.dumps({"identity": ident}))
        self.lock = threading.Lock()
        self.done: dict[tuple[str, int], dict] = {}
        if os.path.exists(self.path):
            with open(self.path) as f:
                for line in filter(str.strip, f):
                    try:
                        rec = json.loads(line)
                    except ValueError:  # a line torn by a kill: that sample runs again
                        continue
                    self.done[(rec["id"], int(rec["repeat"]))] = rec

    def add(self, rec: dict) -> None:
        with self.lock:
            self.done[(rec["id"], int(rec["repeat"]))] = rec
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")

    def scores(self) -> dict[str, list[float]]:
        out: dict[str, list[float]] = {}
        for (i, _), rec in sorted(self.done.items()):
            out.setdefault(i, []).append(float(rec["score"]))
        return out


def load_picture(path: str, multiple: int, max_pixels: int = 1 << 20, min_pixels: int = 0):
    """A picture file as uint8 ``[H, W, 3]`` at :func:`picture_size` (bicubic)."""
    import numpy as np
    from PIL import Image

    img = Image.open(path).convert("RGB")
    w, h = img.size
    h2, w2 = picture_size(h, w, multiple, min_pixels, max_pixels)
    if (w2, h2) != (w, h):
        img = img.resize((w2, h2), Image.BICUBIC)
    return np.asarray(img, dtype=np.uint8)


class BenchmarkRun:
    DONE = "ok"

    def __init__(self, config, router: LeastInFlightRouter, tokenizer, model_name: str, out_dir: str, dataset_dir: str,
                 only: Optional[list[str]] = None, limit: Optional[int] = None, vision=None, hidden_size: int = 0):
        """``vision``: a ``loop.vision_encoder.VisionEncoder`` for items that carry pictures (``"images": [file, ...]`` relative to
        the dataset directory): the pictures follow the question in the user turn, their rows travel with the request."""
        self.config, self.router, self.tok, self.model_name = config, router, tokenizer, model_name
        self.out_dir, self.dataset_dir, self.only, self.limit = out_dir, dataset_dir, only, limit
        self.vision, self.hidden_size = vision, hidden_size
        self.sampling = {k: config["sampling"][k] for k in sorted(config["sampling"])}

    def params(self, max_tokens: int) -> SamplingParams:
        s = self.sampling
        return SamplingParams(max_tokens=max_tokens, temperature=float(s.get("temperature", 1.0)), top_p=float(s.get("top_p", 1.0)),
                              top_k=int(s.get("top_k", 0)), stop_token_ids=(self.tok.eos_id,) + tuple(getattr(self.tok, "extra_stop_ids", ())))

    def _prompt(self, item: Item):
        """(token ids, picture rows [T, hidden] or None, their mask)."""
        files = item.extra.get("images") or []
        if not files:
            return self.tok.render_turn("user", item.prompt) + self.tok.generation_prompt(), None, None
        if self.vision is None:
            raise ValueError(f"item {item.id} carries pictures: the run needs a vision tower (--vision)")
        import torch

        cfg = self.vision.tower.cfg
        multiple = getattr(cfg, "patch_size", getattr(cfg, "patch", 1)) * getattr(cfg, "spatial_merge_size", getattr(cfg, "merge", 1))
        blocks = self.vision.encode([load_picture(os.path.join(self.dataset_dir, f), multiple, int(self.config.get("image_max_pixels", 1 << 20)), int(self.config.get("image_min_pixels", 0))) for f in files])
        ids = self.tok.render_turn("user", item.prompt, images=len(blocks), image_tokens=[b.shape[0] for b in blocks]) + self.tok.generation_prompt()
        mask = torch.tensor([t == self.tok.image_pad_id for t in ids])
        rows = torch.from_numpy(__import__("numpy").concatenate(blocks, axis=0))
        if int(mask.sum()) != rows.shape[0]:
            raise ValueError(f"item {item.id}: {rows.shape[0]} picture rows for {int(mask.sum())} placeholder tokens")
        embeds = torch.zeros(len(ids), rows.shape[1])
        embeds[mask] = rows
        return ids, embeds, mask

    def sample(self, store: SampleStore, bench: dict, item: Item, repeat: int) -> None:
        prompt, embeds, mask = self._prompt(item)
        req = self.router.generate(prompt, self.params(int(bench["max_tokens"])), embeds=embeds, embeds_mask=mask)
        text = self.tok.decode([t for t in req.output if t != self.tok.eos_id], skip_special=True)
        finish = req.finish.value if isinstance(req.finish, FinishReason) else str(req.finish)
        score = scorers.KINDS[bench["kind"]](text, item.as_dict())
        store.add({"id": item.id, "repeat": repeat, "score": float(score), "tokens": len(req.output), "finish": finish, "completion": text})

    def run(self) -> dict[str, dict]:
        """Returns {benchmark: {"status", "mean", "samples", "seconds"}}; raises SystemExit naming the failed benchmarks."""
        names = self.only or list(self.config["benchmarks"])
        os.makedirs(self.out_dir, exist_ok=True)
        report: dict[str, dict] = {}
        jobs, stores, t0 = [], {}, time.monotonic()
        for name in names:
            bench = dict(self.config["benchmarks"][name])
            try:
                if bench["kind"] not in scorers.KINDS:
                    raise ValueError(f"unknown kind {bench['kind']!r}")
                items = load_benchmark(os.path.join(self.dataset_dir, str(bench["file"])), self.limit)
                stores[name] = SampleStore(self.out_dir, name, identity(bench, self.sampling, self.model_name))
                todo = [(name, bench, it, r) for it in items for r in range(int(bench["repeats"])) if (it.id, r) not in stores[name].done]
                report[name] = {"status": self.DONE, "reused": len(items) * int(bench["repeats"]) - len(todo)}
                jobs += todo
            except Exception as e:  # noqa: BLE001 - one benchmark's failure must not stop the others
                report[name] = {"status": f"failed: {e!r}"[:300]}
        # all benchmarks at once, interleaved: round-robin over the benchmarks so that none waits for another's tail
        by_name: dict[str, list] = {}
        for j in jobs:
            by_name.setdefault(j[0], []).append(j)
        order = [q[i] for i in range(max((len(q) for q in by_name.values()), default=0)) for q in by_name.values() if i < len(q)]

        def one(job) -> None:
            name, bench, item, repeat = job
            if report[name]["status"] != self.DONE:
                return
            try:
                self.sample(stores[name], bench, item, repeat)
            except Exception as e:  # noqa: BLE001
                report[name]["status"] = f"failed: {e!r}"[:300]

        with ThreadPoolExecutor(max_workers=int(self.config["concurrency"])) as pool:
            list(pool.map(one, order))
        for name, store in stores.items():
            sc = store.scores()
            report[name].update(samples=len(sc), mean=(sum(sum(v) / len(v) for v in sc.values()) / len(sc)) if sc else 0.0,
                                seconds=time.monotonic() - t0)
            atomic_write(os.path.join(store.dir, "report.json"), json.dumps(report[name]))
        failed = [n for n in names if report[n]["status"] != self.DONE]
        for n in names:
            print(f"{n}: {report[n]['status']}" + (f" mean {100 * report[n]['mean']:.1f} over {report[n]['samples']} items ({report[n]['reused']} samples reused)"
                                                    if "mean" in report[n] else ""), flush=True)
        if failed:
            raise SystemExit(f"{len(failed)} of {len(names)} benchmarks failed: {', '.join(failed)}")
        return report


def dataset_status(config, dataset_dir: str, only: Optional[list[str]] = None) -> dict[str, dict]:
    out = {}
    for name in only or list(config["benchmarks"]):
        bench = config["benchmarks"][name]
        path = os.path.join(dataset_dir, str(bench["file"]))
        if os.path.exists(path):
            items = load_benchmark(path)
            out[name] = {"present": True, "items": len(items), "kind": bench["kind"]}
        else:
            out[name] = {"present": False, "file": path, "source": bench.get("source", "")}
    return out


# -- comparison ---------------------------------------------------------------------------------------------------------------
def mean_se(values: list[float]) -> tuple[float, float]:
    n = len(values)
    m = sum(values) / n
    return m, (sum((v - m) ** 2 for v in values) / max(n - 1, 1) / n) ** 0.5


def paired_bootstrap(a: dict[str, list[float]], b: dict[str, list[float]], samples: int = 10000, seed: int = 0, confidence: float = 0.95) -> dict:
    """Items both runs answered (each item's score = the mean over its repeats), resampled with replacement: mean difference
    b - a, its confidence interval, P(b > a)."""
    ids = sorted(set(a) & set(b))
    if not ids:
        raise ValueError("the runs share no items")
    da = [sum(a[i]) / len(a[i]) for i in ids]
    db = [sum(b[i]) / len(b[i]) for i in ids]
    diff = [y - x for x, y in zip(da, db)]
    rng = random.Random(seed)
    n = len(ids)
    means = sorted(sum(diff[rng.randrange(n)] for _ in range(n)) / n for _ in range(samples))
    tail = int(samples * (1 - confidence) / 2)
    lo, hi = means[tail], means[samples - 1 - tail]
    (ma, sa), (mb, sb) = mean_se(da), mean_se(db)
    return {"items": n, "mean_a": ma, "se_a": sa, "mean_b": mb, "se_b": sb, "diff": sum(diff) / n, "ci95": [lo, hi], "ci": [lo, hi],
            "significant": hi < 0 or lo > 0, "p_b_better": sum(m > 0 for m in means) / samples}


def load_samples(run_dir: str, name: str) -> dict[str, list[float]]:
    path = os.path.join(run_dir, name, "samples.jsonl")
    out: dict[str, list[float]] = {}
    if os.path.exists(path):
        with open(path) as f:
            for line in filter(str.strip, f):
                try:
                    rec = json.loads(line)
                except ValueError:
                    continue
                out.setdefault(rec["id"], []).append(float(rec["score"]))
    return out


def compare_runs(config, run_a: str, run_b: str, names=("a", "b")) -> list[str]:
    bs = config["bootstrap"]
    lines = [f"{'benchmark':22s} {names[0]:>16s} {names[1]:>16s} {'diff':>8s} {'%d%% CI (paired bootstrap)' % round(100 * float(bs['confidence'])):>28s}  n"]
    for name in config["benchmarks"]:
        a, b = load_samples(run_a, name), load_samples(run_b, name)
        if not (set(a) & set(b)):
            lines.append(f"{name:22s} (missing in {'a' if not a else 'b' if not b else 'both: no shared items'})")
            continue
        r = paired_bootstrap(a, b, int(bs["samples"]), int(bs["seed"]), float(bs["confidence"]))
        lines.append(f"{name:22s} {100 * r['mean_a']:9.1f} ±{100 * r['se_a']:4.1f} {100 * r['mean_b']:9.1f} ±{100 * r['se_b']:4.1f} "
                     f"{100 * r['diff']:+8.1f}    [{100 * r['ci'][0]:+6.1f}, {100 * r['ci'][1]:+6.1f}]{' *' if r['significant'] else '  '} {r['items']}")
    lines.append("* the interval of the paired difference excludes 0")
    return lines


def save_run(path: str, scores: dict[str, list[float]]) -> None:
    atomic_write(path, json.dumps(scores))


def load_run(path: str) -> dict[str, list[float]]:
    with open(path) as f:
        return json.load(f)


# -- router process -----------------------------------------------------------------------------------------------------------
def router_app(backends: list[str]):
    """aiohttp application: every request goes to the backend with the fewest requests in flight; the response is streamed back."""
    import aiohttp
    from aiohttp import web

    inflight = [0] * len(backends)

    async def open_session(app):
        app["session"] = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None))

    async def close_session(app):
        await app["session"].close()

    async def proxy(request: web.Request) -> web.StreamResponse:
        i = min(range(len(backends)), key=lambda j: inflight[j])
        inflight[i] += 1
        try:
            body = await request.read()
            async with request.app["session"].request(request.method, backends[i].rstrip("/") + request.rel_url.path_qs, data=body or None,
                                                      headers={k: v for k, v in request.headers.items() if k.lower() not in ("host", "content-length")}) as r:
                resp = web.StreamResponse(status=r.status, headers={k: v for k, v in r.headers.items() if k.lower() in ("content-type",)})
                await resp.prepare(request)
                async for chunk in r.content.iter_any():
                    await resp.write(chunk)
                await resp.write_eof()
                return resp
        finally:
            inflight[i] -= 1

    app = web.Application(client_max_size=1 << 30)
    app["inflight"] = inflight
    app.on_startup.append(open_session)
    app.on_cleanup.append(close_session)
    app.router.add_route("*", "/{tail:.*}", proxy)
    return app


# -- command line -------------------------------------------------------------------------------------------------------------
def main(argv=None) -> int:
    import argparse

    from ..config.loader import compose
    from ..utils.tokenizer import load_tokenizer

    ap = argparse.ArgumentParser(description="general-capability evaluation")
    sub = ap.add_subparsers(dest="command", required=True)
    r = sub.add_parser("run")
    r.add_argument("--replicas", default="", help="url,url,... of rollout replica processes")
    r.add_argument("--model", default="", help="model directory or preset:<name> for in-process replicas (when --replicas is empty)")
    r.add_argument("--num-replicas", type=int, default=1)
    r.add_argument("--vision", default="", help="vision tower for items with pictures: checkpoint (the --model directory's), family_tiny, tiny")
    r.add_argument("--tokenizer", default="", help="directory with the model's tokenizer.json (default: --model; the byte tokenizer without one)")
    r.add_argument("--model-name", default="", help="the name the samples are kept under (default: --model or the first replica URL)")
    r.add_argument("--out", required=True)
    r.add_argument("--dataset-dir", required=True)
    r.add_argument("--only", nargs="+")
    r.add_argument("--limit", type=int, help="a smoke: the first N items of each benchmark")
    d = sub.add_parser("datasets")
    d.add_argument("--dataset-dir", required=True)
    d.add_argument("--only", nargs="+")
    ro = sub.add_parser("router")
    ro.add_argument("--port", type=int, required=True)
    ro.add_argument("--backends", required=True, help="url,url,...")
    c = sub.add_parser("compare")
    c.add_argument("--a", required=True)
    c.add_argument("--b", required=True)
    c.add_argument("--names", nargs=2, default=("a", "b"))
    args, overrides = ap.parse_known_args(argv)
    only = getattr(args, "only", None)
    if only:  # `--only a b key=value`: the list takes everything after it
        overrides += [o for o in only if "=" in o]
        args.only = [o for o in only if "=" not in o] or None
    cfg = compose("general", [o for o in overrides if "=" in o])

    if args.command == "datasets":
        st = dataset_status(cfg, args.dataset_dir, args.only)
        for name, s in st.items():
            print(f"{name}: " + (f"{s['items']} items ({s['kind']})" if s["present"] else f"missing {s['file']} (source: {s['source']})"))
        return 0 if all(s["present"] for s in st.values()) else 1
    if args.command == "router":
        from aiohttp import web

        web.run_app(router_app(args.backends.split(",")), host="127.0.0.1", port=args.port, print=None)
        return 0
    if args.command == "compare":
        print("\n".join(compare_runs(cfg, args.a, args.b, tuple(args.names))))
        return 0

    servers, local = [], []
    if args.replicas:
        from ..rollout.remote import RemoteReplica

        servers = [RemoteReplica(u, name=f"replica-{i}") for i, u in enumerate(args.replicas.split(","))]
        for s in servers:
            s.wait_ready()
    else:
        from ..rollout.engine import EngineConfig
        from ..rollout.server import build_server, load_rollout_model

        if not args.model:
            ap.error("run needs --replicas or --model")
        for i in range(args.num_replicas):
            local.append(build_server(load_rollout_model(args.model, with_mtp=False), EngineConfig(), name=f"replica-{i}"))
        servers = local
    vision = None
    if args.vision:
        from ..loop.vision_encoder import build_vision_encoder

        try:
            vision = build_vision_encoder(args.vision, args.model)
        except ValueError as e:
            ap.error(str(e))
    try:
        BenchmarkRun(cfg, LeastInFlightRouter(servers), load_tokenizer(args.tokenizer or args.model), args.model_name or args.model or args.replicas.split(",")[0],
                     args.out, args.dataset_dir, args.only, args.limit, vision=vision).run()
    finally:
        for s in servers:
            s.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
