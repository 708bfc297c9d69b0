"""General benchmark evaluation (upstream ``pear/eval/general.py:16-353``): a least-in-flight router over rollout
replicas, a benchmark = a list of (prompt, checker) items generated ``n`` times each, and a PAIRED bootstrap
comparison of two runs over the same items (the protocol of ``configs/general.yaml``).

Benchmarks are plain JSONL files (``{"id", "prompt", "answer"}``) — no benchmark suite is bundled; the scorer is exact
match of the last line of the completion unless a callable is given."""

from __future__ import annotations

import json
import os
import random
import threading
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from typing import Callable, Optional

from ..rollout.engine import SamplingParams
from ..utils.files import atomic_write


class LeastInFlightRouter:
    def __init__(self, servers: list):
        self.servers, self.inflight, self.lock = servers, [0] * len(servers), threading.Lock()

    def generate(self, prompt: list[int], params: SamplingParams):
        with self.lock:
            i = min(range(len(self.servers)), key=lambda j: self.inflight[j])
            self.inflight[i] += 1
        try:
            return self.servers[i].generate(prompt, params)
        finally:
            with self.lock:
                self.inflight[i] -= 1


@dataclass
class Item:
    id: str
    prompt: str
    answer: str


def load_benchmark(path: str) -> list[Item]:
    with open(path) as f:
        return [Item(str(d["id"]), d["prompt"], str(d["answer"])) for d in map(json.loads, f) if d]


def exact_last_line(completion: str, answer: str) -> float:
    lines = [l.strip() for l in completion.strip().splitlines() if l.strip()]
    return float(bool(lines) and lines[-1] == answer.strip())


def run_benchmark(router: LeastInFlightRouter, tokenizer, items: list[Item], n: int = 1, temperature: float = 1.0, top_p: float = 0.95,
                  max_tokens: int = 256, scorer: Callable[[str, str], float] = exact_last_line, workers: int = 16) -> dict[str, list[float]]:
    params = SamplingParams(max_tokens=max_tokens, temperature=temperature, top_p=top_p, stop_token_ids=(tokenizer.eos_id,))

    def one(item: Item) -> tuple[str, list[float]]:
        prompt = tokenizer.render_turn("user", item.prompt) + tokenizer.generation_prompt()
        scores = []
        for _ in range(n):
            req = router.generate(prompt, params)
            scores.append(scorer(tokenizer.decode([t for t in req.output if t != tokenizer.eos_id], skip_special=True), item.answer))
        return item.id, scores

    with ThreadPoolExecutor(max_workers=workers) as ex:
        return dict(ex.map(one, items))


def paired_bootstrap(a: dict[str, list[float]], b: dict[str, list[float]], samples: int = 10000, seed: int = 0) -> dict:
    """Items both runs answered, resampled with replacement: mean difference b - a, its 95% interval, P(b > a)."""
    ids = sorted(set(a) & set(b))
    if not ids:
        raise ValueError("the runs share no items")
    da = [sum(a[i]) / len(a[i]) for i in ids]
    db = [sum(b[i]) / len(b[i]) for i in ids]
    diff = [y - x for x, y in zip(da, db)]
    rng = random.Random(seed)
    n = len(ids)
    means = sorted(sum(diff[rng.randrange(n)] for _ in range(n)) / n for _ in range(samples))
    return {"items": n, "mean_a": sum(da) / n, "mean_b": sum(db) / n, "diff": sum(diff) / n,
            "ci95": [means[int(0.025 * samples)], means[min(samples - 1, int(0.975 * samples))]],
            "p_b_better": sum(m > 0 for m in means) / samples}


def save_run(path: str, scores: dict[str, list[float]]) -> None:
    atomic_write(path, json.dumps(scores))


def load_run(path: str) -> dict[str, list[float]]:
    with open(path) as f:
        return json.load(f)


def main(argv=None) -> int:
    import sys

    from ..config.loader import compose
    from ..models import io as model_io
    from ..models.hybrid import HybridForCausalLM
    from ..rollout.engine import EngineConfig
    from ..rollout.server import build_server
    from ..utils.tokenizer import ByteTokenizer

    cfg = compose("general", list(sys.argv[1:] if argv is None else argv))
    mcfg = model_io.load_config(str(cfg.model))
    servers = []
    for i in range(int(cfg.replicas)):
        m = HybridForCausalLM(mcfg, with_mtp=False)
        model_io.load_model_dir(str(cfg.model), m)
        servers.append(build_server(m, EngineConfig(), name=f"replica-{i}"))
    tok = ByteTokenizer()
    os.makedirs(str(cfg.run_dir), exist_ok=True)
    try:
        router = LeastInFlightRouter(servers)
        g = cfg.generation
        for bench in cfg.benchmarks:
            scores = run_benchmark(router, tok, load_benchmark(str(bench)), int(g.n), float(g.temperature), float(g.top_p), int(g.max_tokens))
            name = os.path.splitext(os.path.basename(str(bench)))[0]
            save_run(os.path.join(str(cfg.run_dir), f"{name}.json"), scores)
            report = {"benchmark": name, "mean": sum(sum(v) / len(v) for v in scores.values()) / max(1, len(scores))}
            if cfg.compare.baseline:
                report["vs_baseline"] = paired_bootstrap(load_run(os.path.join(str(cfg.compare.baseline), f"{name}.json")), scores,
                                                         int(cfg.compare.bootstrap_samples), int(cfg.compare.seed))
            print(json.dumps(report))
    finally:
        for s in servers:
            s.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
