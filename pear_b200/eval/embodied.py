"""Embodied evaluation: a training rollout without training (upstream ``pear/eval/embodied.py:24-222``).

Runs every episode row ``n`` times through the agent loop against the rollout replicas, records each finished group to
``eval_<step>.jsonl`` and writes a summary (success rate per family and per task, end reasons, turns, tokens)."""

from __future__ import annotations

import json
import os
import sys
from collections import Counter, defaultdict
from typing import Optional

from ..loop.agent_loop import AgentLoopConfig
from ..loop.dataset import EpisodeDataset
from ..loop.manager import AgentLoopManager
from ..loop.transfer_queue import TransferQueue
from ..utils.files import append_jsonl, atomic_write


def evaluate(servers: list, hidden_size: int, env_families: dict, episodes, output_dir: str, step: int = 0, n: int = 1,
             loop_cfg: Optional[AgentLoopConfig] = None, num_workers: int = 4, timeout_s: float = 3600.0) -> dict:
    os.makedirs(output_dir, exist_ok=True)
    ds = EpisodeDataset(episodes, shuffle=False)
    queue = TransferQueue(4)
    mgr = AgentLoopManager(servers, hidden_size, env_families, loop_cfg or AgentLoopConfig(), queue, num_workers=num_workers)
    out_path = os.path.join(output_dir, f"eval_{step}.jsonl")
    by_family: dict[str, list[float]] = defaultdict(list)
    by_task: dict[str, list[float]] = defaultdict(list)
    ends: Counter = Counter()
    turns, tokens = [], []
    try:
        futs = [(row, mgr.dispatch_group(f"eval-{row.index}", row.family, row.env_args, [str(i) for i in range(n)])) for row in ds.rows]
        for row, fs in futs:
            eps = [f.result(timeout=timeout_s) for f in fs]
            rewards = [float(e.success) for e in eps]
            append_jsonl(out_path, {"index": row.index, "family": row.family, "env_args": row.env_args, "rewards": rewards,
                                    "end_reasons": [e.end_reason.value if e.end_reason else None for e in eps],
                                    "turns": [e.turns for e in eps], "tokens": [len(e.tokens) for e in eps]})
            by_family[row.family] += rewards
            by_task[f"{row.family}/{row.env_args.get('task', '-')}"] += rewards
            for e in eps:
                ends[e.end_reason.value if e.end_reason else "none"] += 1
                turns.append(e.turns)
                tokens.append(len(e.tokens))
            queue.clear_prefix(f"eval-{row.index}/")
    finally:
        mgr.close()
    mean = lambda xs: sum(xs) / max(1, len(xs))  # noqa: E731
    summary = {"step": step, "episodes": len(ds.rows), "n": n, "success_rate": mean([r for v in by_family.values() for r in v]),
               "families": {k: mean(v) for k, v in sorted(by_family.items())}, "tasks": {k: mean(v) for k, v in sorted(by_task.items())},
               "end_reasons": dict(ends), "mean_turns": mean(turns), "mean_tokens": mean(tokens)}
    atomic_write(os.path.join(output_dir, f"summary_{step}.json"), json.dumps(summary, indent=1))
    return summary


def main(argv=None) -> int:
    from ..config.loader import compose
    from ..models import io as model_io
    from ..models.config import HybridConfig
    from ..models.hybrid import HybridForCausalLM
    from ..rollout.engine import EngineConfig
    from ..rollout.server import build_server

    cfg = compose("embodied", list(sys.argv[1:] if argv is None else argv))
    path = str(cfg.actor_rollout_ref.model.path)
    mcfg = getattr(HybridConfig, path.split(":", 1)[1])() if path.startswith("preset:") else model_io.load_config(path)
    model = HybridForCausalLM(mcfg, with_mtp=False)
    if path.startswith("preset:"):
        model.init_weights(0)
    else:
        model_io.load_model_dir(path, model)
    ro = cfg.actor_rollout_ref.rollout
    server = build_server(model, EngineConfig(max_num_seqs=int(ro.max_num_seqs), block_size=int(ro.block_size)))
    try:
        families = {"synthetic": {"env_path": "pear_b200.envs.synthetic.SyntheticEnv", "env_kwargs": {"hidden": mcfg.hidden_size}}}
        s = evaluate([server], mcfg.hidden_size, families, cfg.eval.episodes, str(cfg.eval.output_dir), n=int(cfg.eval.n),
                     loop_cfg=AgentLoopConfig(token_budget=int(cfg.data.max_response_length), temperature=float(ro.temperature), top_p=float(ro.top_p)))
        print(json.dumps(s))
    finally:
        server.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
