"""Tool-call parser registry (upstream ``pear/agent_loop/tool_parser.py:11-57`` and the model family's
``tool_parser.py:5-9``): a parser turns a decoded answer into tool calls; the family registers its own by name."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .protocol import ParseError, extract_action


@dataclass
class ToolCall:
    name: str
    arguments: dict


_PARSERS: dict[str, Callable[[str], list[ToolCall]]] = {}


def register(name: str):
    def deco(fn):
        _PARSERS[name] = fn
        return fn
    return deco


def get_parser(name: str) -> Callable[[str], list[ToolCall]]:
    if name not in _PARSERS:
        raise KeyError(f"unknown tool parser {name!r}; registered: {sorted(_PARSERS)}")
    return _PARSERS[name]


@register("fenced_json")
def fenced_json(text: str) -> list[ToolCall]:
    """One call to the environment tool per answer; an unparsable answer gives no call (the loop ends with PARSE)."""
    try:
        return [ToolCall("env", extract_action(text))]
    except ParseError:
        return []


# the hybrid GDN + attention family answers in the same format (`multi_turn.format` of the recipes names it)
register("qwen3_5")(fenced_json)
register("qwen3_8")(fenced_json)
