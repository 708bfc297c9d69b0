"""Monitor (metrics scraper, tracker, driver log, panel) and evaluation helpers on CPU."""

import json
import os

import torch

from pear_b200.eval.general import Item, LeastInFlightRouter, paired_bootstrap, run_benchmark
from pear_b200.models.config import HybridConfig
from pear_b200.models.hybrid import HybridForCausalLM
from pear_b200.monitor.driver_log import DriverLog
from pear_b200.monitor.metrics import MetricsScraper, parse_prometheus
from pear_b200.monitor.progress_panel import ProgressPanel
from pear_b200.monitor.progress_tracker import ProgressTracker
from pear_b200.rollout.engine import EngineConfig, SamplingParams
from pear_b200.rollout.server import build_server
from pear_b200.utils.tokenizer import ByteTokenizer


def test_prometheus_parse_and_rates():
    text = '# TYPE x counter\npear_generation_tokens_total{replica="a"} 10\npear_num_running{replica="a"} 2\n'
    assert parse_prometheus(text) == {"pear_generation_tokens_total": 10.0, "pear_num_running": 2.0}
    vals = {"n": 0}

    def src():
        vals["n"] += 100
        return f'pear_generation_tokens_total{{replica="a"}} {vals["n"]}\npear_num_running{{replica="a"}} 1\n'

    def dead():
        raise ConnectionError("down")

    s = MetricsScraper({"a": src, "b": dead})
    s.scrape()
    s.last["a"].t -= 2.0  # two seconds ago
    s.scrape()
    assert 40 < s.rates()["a"]["pear_generation_tokens_per_s"] < 60
    assert "b" in s.errors and s.summary()["pear_num_running"] == 1.0


def test_tracker_driver_log_and_panel(tmp_path):
    tr = ProgressTracker()
    tr.record("g", "0", "synthetic", 1.0, 3, "env", 100)
    tr.record("g", "1", "synthetic", 0.0, 5, "parse", 50)
    snap = tr.snapshot()
    assert snap["families"]["synthetic"]["success_rate"] == 0.5 and snap["end_reasons"] == {"env": 1, "parse": 1}
    log = tmp_path / "train.log"
    log.write_text("noise\nstep:1 - timing/train_s:2.5 - data/reward_mean:0.25 - timing/wait_rollout_s:1\nstep:2 - timing/train_s:3")
    d = DriverLog(str(log))
    assert [r.step for r in d.poll()] == [1] and d.latest().phases == {"train_s": 2.5, "wait_rollout_s": 1.0}
    with open(log, "a") as f:
        f.write(".5\n")
    assert [r.step for r in d.poll()] == [2] and d.latest().phases["train_s"] == 3.5
    panel = ProgressPanel(str(tmp_path), MetricsScraper({"a": lambda: "pear_num_running 1\n"}), tr)
    state = panel.tick()
    assert state["trainer"]["step"] == 2 and json.load(open(tmp_path / "progress.json"))["trajectories"]["episodes"] == 2
    assert "episodes 2" in open(tmp_path / "progress.log").read()


def test_paired_bootstrap():
    a = {str(i): [0.0] for i in range(40)}
    b = {str(i): [1.0 if i % 2 else 0.0] for i in range(40)}
    r = paired_bootstrap(a, b, samples=500, seed=1)
    assert r["items"] == 40 and abs(r["diff"] - 0.5) < 1e-9 and r["p_b_better"] == 1.0 and r["ci95"][0] > 0.2


def test_server_metrics_pause_resubmit_and_benchmark():
    cfg = HybridConfig.tiny()
    model = HybridForCausalLM(cfg, with_mtp=False).init_weights(0)
    srv = build_server(model, EngineConfig(num_blocks=256, max_num_seqs=4))
    try:
        tok = ByteTokenizer()
        router = LeastInFlightRouter([srv])
        scores = run_benchmark(router, tok, [Item("0", "2+2?", "4"), Item("1", "3+3?", "6")], n=2, max_tokens=8, workers=2)
        assert set(scores) == {"0", "1"} and all(len(v) == 2 for v in scores.values())
        text = srv.metrics_text()
        assert "pear_generation_tokens_total" in text
        vals = {l.split("{")[0]: float(l.split()[-1]) for l in text.splitlines() if l and not l.startswith("#")}
        assert vals["pear_requests_finished_total"] == 4 and vals["pear_first_tokens_total"] == 4  # 2 items x 2 samples
        assert vals["pear_request_seconds_total"] >= vals["pear_first_token_seconds_total"] > 0
        # a paused replica rejects new requests as aborted; generate() resubmits after the resume
        srv.pause(abort=True)
        fut = srv.submit([1, 2, 3], SamplingParams(max_tokens=4))
        assert fut.result(timeout=5).finish.value == "aborted"
        srv.update_weights({k: v.detach().clone() for k, v in model.state_dict().items()}, version=7)
        srv.resume()
        req = srv.generate([1, 2, 3], SamplingParams(max_tokens=4), timeout_s=60)
        assert len(req.output) == 4 and req.policy_version == 7
    finally:
        srv.close()


def test_chat_completions_endpoint_renders_the_template():
    from fastapi.testclient import TestClient

    cfg = HybridConfig.tiny()
    srv = build_server(HybridForCausalLM(cfg, with_mtp=False).init_weights(0), EngineConfig(num_blocks=128, max_num_seqs=4))
    try:
        tok = ByteTokenizer()
        client = TestClient(srv.http_app(tok))
        body = {"model": "m", "messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": [{"type": "text", "text": "2+2?"}]}],
                "max_tokens": 5, "temperature": 0.0, "n": 2}
        out = client.post("/v1/chat/completions", json=body).json()
        assert out["object"] == "chat.completion" and len(out["choices"]) == 2 and out["choices"][0]["message"]["role"] == "assistant"
        want_prompt = tok.render_turn("system", "be brief") + tok.render_turn("user", "2+2?") + tok.generation_prompt()
        assert out["usage"]["prompt_tokens"] == len(want_prompt) and 0 < out["usage"]["completion_tokens"] <= 10
        direct = srv.generate(want_prompt, SamplingParams(max_tokens=5, temperature=0.0, stop_token_ids=(tok.eos_id,)))
        assert out["choices"][0]["message"]["content"] == tok.decode([t for t in direct.output if t != tok.eos_id], skip_special=True)
        assert out["choices"][0]["message"]["content"] == out["choices"][1]["message"]["content"]  # greedy twice
        assert "error" in TestClient(srv.http_app()).post("/v1/chat/completions", json=body).json()
    finally:
        srv.close()


def test_monitor_derives_cache_hit_rate_and_latencies_from_replica_counters():
    def text(q, h, x, n, secs, gen):
        vals = {"pear_prefix_cache_queries_total": q, "pear_prefix_cache_hits_total": h, "pear_external_prefix_cache_hits_total": x,
                "pear_requests_finished_total": n, "pear_request_seconds_total": secs, "pear_generation_tokens_total": gen}
        return "\n".join(f'{k}{{replica="r"}} {float(v)}' for k, v in vals.items()) + "\n"

    feeds = iter([text(0, 0, 0, 0, 0.0, 0), text(1000, 600, 100, 10, 25.0, 500)])
    sc = MetricsScraper({"r": "http://unused"})
    sc._fetch = lambda src: next(feeds)
    sc.scrape()
    import time
    time.sleep(0.05)
    sc.scrape()
    s = sc.summary()
    assert abs(s["cache_hit_rate"] - 0.6) < 1e-9 and abs(s["external_cache_hit_rate"] - 0.1) < 1e-9 and abs(s["mean_request_seconds"] - 2.5) < 1e-9
    assert s["pear_generation_tokens_per_s"] > 0
