"""Reads the action out of a model's complete final answer, strictly: the answer must end with one fenced json block holding
exactly the format's parts and quantities as finite numbers; an answer with a thinking block, trailing text, a repeated key,
a boolean or an out-of-bounds quantity is refused (ValueError), so nothing half-understood reaches a robot. The rules are
upstream's (pear/deploy/station/agent_loop/action_parser.py:10-49); bounds are this format's own addition."""

from __future__ import annotations

import json
import math
import re

from .robot import ActionFormat

THINK_START = "<think>"
JSON_BLOCK = re.compile(r"```json\s*\n(.*?)\n\s*```", re.DOTALL)


def _unique(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise ValueError(f"Duplicate action field: {k}")
        out[k] = v
    return out


def parse_action(answer: str, fmt: ActionFormat) -> dict:
    if THINK_START in answer:
        raise ValueError("Final answer unexpectedly contains a thinking block")
    blocks = list(JSON_BLOCK.finditer(answer))
    if not blocks or answer[blocks[-1].end():].strip():
        raise ValueError("Final answer must end with a fenced json action")
    try:
        fields = json.loads(blocks[-1].group(1), object_pairs_hook=_unique)
    except json.JSONDecodeError as e:
        raise ValueError(f"The action is not valid JSON: {e}") from e
    if not isinstance(fields, dict) or set(fields) != set(fmt.schema):
        raise ValueError("Expected exactly the parts " + ", ".join(fmt.schema))
    for part, names in fmt.schema.items():
        q = fields[part]
        if not isinstance(q, dict) or set(q) != set(names):
            raise ValueError(f"Invalid quantities for {part}")
        for name, v in q.items():
            if type(v) not in (int, float) or not math.isfinite(v):
                raise ValueError("Action quantities must be finite numbers, not booleans")
            lo, hi = fmt.bounds.get(f"{part}.{name}", (-math.inf, math.inf))
            if not lo <= v <= hi:
                raise ValueError(f"{part}.{name} = {v} is outside [{lo}, {hi}]")
    return fields
