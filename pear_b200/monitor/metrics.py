"""Replica metrics scraper (upstream ``pear/monitor/metrics.py:84-233``): polls every replica's Prometheus exposition
(the text of ``RolloutServer.metrics_text`` or an HTTP ``/metrics`` URL), keeps the last two samples per replica and
turns counters into rates."""

from __future__ import annotations

import re
import time
import urllib.request
from dataclasses import dataclass, field
from typing import Callable, Optional, Union

COUNTERS = ("pear_prompt_tokens_total", "pear_generation_tokens_total", "pear_preemptions_total", "pear_aborted_total",
            "pear_spec_drafted_total", "pear_spec_accepted_total", "pear_prefix_cache_queries_total", "pear_prefix_cache_hits_total",
            "pear_external_prefix_cache_hits_total", "pear_requests_finished_total", "pear_request_seconds_total", "pear_first_tokens_total",
            "pear_first_token_seconds_total")
GAUGES = ("pear_num_running", "pear_num_waiting", "pear_policy_version", "pear_free_blocks", "pear_cached_blocks")
_LINE = re.compile(r"^([a-zA-Z_:][a-zA-Z0-9_:]*)(\{[^}]*\})?\s+([-+0-9.eE]+|NaN|[+-]?Inf)$")


def parse_prometheus(text: str) -> dict[str, float]:
    out: dict[str, float] = {}
    for line in text.splitlines():
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        m = _LINE.match(line)
        if m:
            out[m.group(1)] = out.get(m.group(1), 0.0) + float(m.group(3))
    return out


@dataclass
class ReplicaSample:
    t: float
    values: dict[str, float]


@dataclass
class MetricsScraper:
    sources: dict[str, Union[str, Callable[[], str]]]   # replica name -> URL or callable returning the exposition text
    timeout_s: float = 2.0
    last: dict[str, ReplicaSample] = field(default_factory=dict)
    prev: dict[str, ReplicaSample] = field(default_factory=dict)
    errors: dict[str, str] = field(default_factory=dict)

    def _fetch(self, src) -> str:
        if callable(src):
            return src()
        with urllib.request.urlopen(src, timeout=self.timeout_s) as r:
            return r.read().decode()

    def scrape(self) -> dict[str, dict[str, float]]:
        now = time.time()
        for name, src in self.sources.items():
            try:
                vals = parse_prometheus(self._fetch(src))
                self.errors.pop(name, None)
            except Exception as e:  # noqa: BLE001 - a dead replica must not stop the monitor
                self.errors[name] = f"{type(e).__name__}: {e}"
                continue
            if name in self.last:
                self.prev[name] = self.last[name]
            self.last[name] = ReplicaSample(now, vals)
        return {n: s.values for n, s in self.last.items()}

    def rates(self) -> dict[str, dict[str, float]]:
        out = {}
        for name, cur in self.last.items():
            p = self.prev.get(name)
            if p is None or cur.t <= p.t:
                continue
            out[name] = {c.replace("_total", "_per_s"): (cur.values.get(c, 0.0) - p.values.get(c, 0.0)) / (cur.t - p.t) for c in COUNTERS}
        return out

    def summary(self) -> dict[str, float]:
        s: dict[str, float] = {}
        for sample in self.last.values():
            for g in GAUGES:
                s[g] = s.get(g, 0.0) + sample.values.get(g, 0.0)
        for r in self.rates().values():
            for k, v in r.items():
                s[k] = s.get(k, 0.0) + v
        d, a = (sum(v.values.get(f"pear_spec_{x}_total", 0.0) for v in self.last.values()) for x in ("drafted", "accepted"))
        if d > 0:
            s["spec_accept_rate"] = a / d
        # share of looked-up prompt tokens found in a cache over the last interval (device tier + host tier), as upstream's panel
        # shows it (monitor/metrics.py:36-42), and the mean request latency / time to first token of that interval
        q = s.get("pear_prefix_cache_queries_per_s", 0.0)
        if q > 0:
            s["cache_hit_rate"] = (s.get("pear_prefix_cache_hits_per_s", 0.0)) / q
            s["external_cache_hit_rate"] = s.get("pear_external_prefix_cache_hits_per_s", 0.0) / q
        for what, count in (("request_seconds", "requests_finished"), ("first_token_seconds", "first_tokens")):
            n = s.get(f"pear_{count}_per_s", 0.0)
            if n > 0:
                s[f"mean_{what}"] = s.get(f"pear_{what}_per_s", 0.0) / n
        s["replicas_up"] = float(len(self.last) - len(self.errors))
        return s
