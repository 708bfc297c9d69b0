"""Answer protocol: the action is the LAST fenced ``json`` block after ``</think>``; it must satisfy the environment's
action schema (upstream ``pear/agent_loop/protocol.py:9-45``, ``tool_parser.py:11-57``)."""

from __future__ import annotations

import json
import re
from typing import Any, Optional

_FENCE = re.compile(r"```json\s*\n(.*?)```", re.DOTALL)


class ParseError(ValueError):
    pass


def extract_action(text: str) -> dict:
    """The last fenced json block after the closing think tag (the whole text when the model did not think)."""
    tail = text.rsplit("</think>", 1)[-1]
    blocks = _FENCE.findall(tail)
    if not blocks:
        raise ParseError("no fenced json block after </think>")
    try:
        obj = json.loads(blocks[-1])
    except json.JSONDecodeError as e:
        raise ParseError(f"invalid json: {e}") from e
    if not isinstance(obj, dict):
        raise ParseError("the action must be a JSON object")
    return obj


def _check(value: Any, schema: dict, path: str) -> Optional[str]:
    t = schema.get("type")
    if t == "object":
        if not isinstance(value, dict):
            return f"{path}: expected object"
        props = schema.get("properties", {})
        for k in schema.get("required", []):
            if k not in value:
                return f"{path}: missing {k!r}"
        if len(value) < schema.get("minProperties", 0):
            return f"{path}: needs at least {schema['minProperties']} properties"
        for k, v in value.items():
            if k in props:
                err = _check(v, props[k], f"{path}.{k}")
                if err:
                    return err
            elif schema.get("additionalProperties", True) is False:
                return f"{path}: unexpected {k!r}"
    elif t == "integer":
        if isinstance(value, bool) or not isinstance(value, int):
            return f"{path}: expected integer"
    elif t == "number":
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            return f"{path}: expected number"
    elif t == "boolean":
        if not isinstance(value, bool):
            return f"{path}: expected boolean"
    elif t == "string":
        if not isinstance(value, str):
            return f"{path}: expected string"
    elif t == "array":
        if not isinstance(value, list):
            return f"{path}: expected array"
        for i, v in enumerate(value):
            err = _check(v, schema.get("items", {}), f"{path}[{i}]")
            if err:
                return err
        if "minItems" in schema and len(value) < schema["minItems"]:
            return f"{path}: too few items"
        if "maxItems" in schema and len(value) > schema["maxItems"]:
            return f"{path}: too many items"
    if "enum" in schema and value not in schema["enum"]:
        return f"{path}: not one of {schema['enum']}"
    if isinstance(value, (int, float)) and not isinstance(value, bool):
        if "minimum" in schema and value < schema["minimum"]:
            return f"{path}: below minimum"
        if "maximum" in schema and value > schema["maximum"]:
            return f"{path}: above maximum"
    return None


def validate_action(action: dict, schema: dict) -> None:
    err = _check(action, schema, "action")
    if err:
        raise ParseError(err)


def parse_answer(text: str, schema: dict) -> dict:
    action = extract_action(text)
    validate_action(action, schema)
    return action
