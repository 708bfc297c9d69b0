"""Scorers of the general-capability protocol: one function per benchmark kind, ``score(completion, item) -> float in [0, 1]``.

Upstream delegates scoring to evalscope's benchmark adapters (``pear/eval/general.py:139-175`` runs each benchmark of
``pear/configs/general.yaml`` as an evalscope task); this build owns them, as small exact rules over the part of the completion
that follows the model's reasoning block:

* ``math_boxed``: the last ``\\boxed{...}`` (else the last number) against the reference, after normalising LaTeX spacing,
  ``\\frac{a}{b}``, thousands separators and trailing zeros (AIME-style integer answers, numeric answers in general);
* ``multiple_choice``: the letter after ``ANSWER:`` / ``answer is`` (else the last stand-alone option letter) against the key
  (GPQA, MMMU, RealWorldQA-style items with lettered options);
* ``instruction_following``: the fraction (or, ``strict``, the conjunction) of the item's verifiable instructions the completion
  satisfies (IFBench-style: word / sentence / paragraph counts, required or forbidden words, case, bullets, JSON, quotation,
  ending phrase, placeholders, sections);
* ``code_stdin``: the last fenced code block run as a Python program on each test's stdin in a child process with a time and
  memory limit; all tests must print the expected stdout (LiveCodeBench's stdin/stdout problems);
* ``exact_last_line``: the last non-empty line equals the answer.
"""

from __future__ import annotations

import json
import math
import os
import re
import subprocess
import sys
import tempfile
from fractions import Fraction
from typing import Callable, Optional

_THINK = re.compile(r"<think>.*?</think>", re.S)


def answer_part(completion: str) -> str:
    """The completion without its reasoning block (an unterminated block leaves nothing to score)."""
    text = _THINK.sub("", completion)
    if "<think>" in text:
        text = text.split("<think>", 1)[0]
    return text.strip()


# -- math ---------------------------------------------------------------------------------------------------------------------
def last_boxed(text: str) -> Optional[str]:
    i = text.rfind("\\boxed")
    if i < 0:
        return None
    j = text.find("{", i)
    if j < 0:
        return None
    depth = 0
    for k in range(j, len(text)):
        if text[k] == "{":
            depth += 1
        elif text[k] == "}":
            depth -= 1
            if depth == 0:
                return text[j + 1:k]
    return None


_FRAC = re.compile(r"\\[dt]?frac\s*\{([^{}]+)\}\s*\{([^{}]+)\}")


def normalize_math(s: str) -> str:
    s = s.strip().strip("$").strip()
    s = re.sub(r"\\text\s*\{([^{}]*)\}", r"\1", s)
    s = re.sub(r"\\(left|right|,|;|!|:| )", "", s)
    s = s.replace("\\%", "").replace("%", "").replace("^\\circ", "").replace("^{\\circ}", "").replace("\\$", "")
    while True:
        m = _FRAC.search(s)
        if not m:
            break
        s = s[:m.start()] + f"({m.group(1)})/({m.group(2)})" + s[m.end():]
    s = s.replace(" ", "").rstrip(".")
    if re.fullmatch(r"-?[\d,]+(\.\d+)?", s):
        s = s.replace(",", "")
    return s


def _as_number(s: str) -> Optional[Fraction]:
    s = s.replace("(", "").replace(")", "")
    try:
        if "/" in s:
            a, b = s.split("/", 1)
            return Fraction(a) / Fraction(b)
        return Fraction(s)
    except (ValueError, ZeroDivisionError):
        return None


def math_boxed(completion: str, item: dict) -> float:
    text = answer_part(completion)
    got = last_boxed(text)
    if got is None:
        nums = re.findall(r"-?\d[\d,]*(?:\.\d+)?(?:/\d+)?", text)
        if not nums:
            return 0.0
        got = nums[-1]
    a, b = normalize_math(got), normalize_math(str(item["answer"]))
    if a == b:
        return 1.0
    na, nb = _as_number(a), _as_number(b)
    if na is not None and nb is not None:
        return float(na == nb or math.isclose(float(na), float(nb), rel_tol=1e-9, abs_tol=1e-12))
    return 0.0


# -- multiple choice ------------------------------------------------------------------------------------------------------------
def multiple_choice(completion: str, item: dict) -> float:
    text = answer_part(completion)
    letters = "ABCDEFGHIJ"[: int(item.get("num_options", 10))]
    m = None
    for pat in (rf"(?i)answer\s*(?:is|:)\s*\**\s*\(?([{letters}])\)?\b", rf"\\boxed\{{\s*\(?([{letters}])\)?\s*\}}"):
        found = re.findall(pat, text)
        if found:
            m = found[-1]
            break
    if m is None:
        found = re.findall(rf"(?<![A-Za-z])\(?([{letters}])\)?(?![A-Za-z])", text)
        m = found[-1] if found else None
    return float(m is not None and m.upper() == str(item["answer"]).strip().upper())


# -- verifiable instructions ----------------------------------------------------------------------------------------------------
def _words(t: str) -> list[str]:
    return re.findall(r"[A-Za-z0-9'-]+", t)


def _relation(n: int, relation: str, target: int) -> bool:
    return {"at least": n >= target, "at most": n <= target, "less than": n < target, "more than": n > target, "exactly": n == target}[relation]


def _is_json(t: str) -> bool:
    t = t.strip()
    t = re.sub(r"^```(?:json)?\s*|\s*```$", "", t)
    try:
        json.loads(t)
        return True
    except ValueError:
        return False


INSTRUCTIONS: dict[str, Callable[[str, dict], bool]] = {
    "length:words": lambda t, a: _relation(len(_words(t)), a["relation"], int(a["n"])),
    "length:sentences": lambda t, a: _relation(len([s for s in re.split(r"(?<=[.!?])\s+", t.strip()) if s]), a["relation"], int(a["n"])),
    "length:paragraphs": lambda t, a: _relation(len([p for p in re.split(r"\n\s*\n", t.strip()) if p.strip()]), a.get("relation", "exactly"), int(a["n"])),
    "keywords:include": lambda t, a: all(re.search(rf"(?i)\b{re.escape(k)}\b", t) for k in a["keywords"]),
    "keywords:exclude": lambda t, a: not any(re.search(rf"(?i)\b{re.escape(k)}\b", t) for k in a["keywords"]),
    "keywords:frequency": lambda t, a: _relation(len(re.findall(rf"(?i)\b{re.escape(a['keyword'])}\b", t)), a["relation"], int(a["n"])),
    "case:lower": lambda t, a: t == t.lower() and any(c.isalpha() for c in t),
    "case:upper": lambda t, a: t == t.upper() and any(c.isalpha() for c in t),
    "format:bullets": lambda t, a: len(re.findall(r"(?m)^\s*[*-]\s+\S", t)) == int(a["n"]),
    "format:json": lambda t, a: _is_json(t),
    "format:quoted": lambda t, a: len(t.strip()) > 1 and t.strip()[0] == '"' and t.strip()[-1] == '"',
    "format:title": lambda t, a: re.search(r"<<[^\n]+>>", t) is not None,
    "format:sections": lambda t, a: len(re.findall(rf"(?m)^\s*{re.escape(a.get('marker', 'SECTION'))}\s+\d+", t)) == int(a["n"]),
    "format:placeholders": lambda t, a: len(re.findall(r"\[[^\[\]]+\]", t)) >= int(a["n"]),
    "content:ends_with": lambda t, a: t.strip().endswith(a["phrase"].strip()),
    "content:starts_with": lambda t, a: t.strip().startswith(a["phrase"].strip()),
    "content:no_commas": lambda t, a: "," not in t,
    "content:postscript": lambda t, a: re.search(rf"(?m)^\s*{re.escape(a.get('marker', 'P.S.'))}", t) is not None,
}


def instruction_following(completion: str, item: dict) -> float:
    text = answer_part(completion)
    checks = item["instructions"]
    if not checks:
        raise ValueError(f"item {item.get('id')}: no instructions")
    passed = []
    for c in checks:
        fn = INSTRUCTIONS.get(c["id"])
        if fn is None:
            raise ValueError(f"item {item.get('id')}: unknown instruction {c['id']!r}")
        passed.append(bool(text) and bool(fn(text, c.get("args", {}))))
    return float(all(passed)) if item.get("strict", True) else sum(passed) / len(passed)


# -- code -----------------------------------------------------------------------------------------------------------------------
def last_code_block(text: str) -> Optional[str]:
    blocks = re.findall(r"```(?:python|py)?\s*\n(.*?)```", text, re.S)
    return blocks[-1] if blocks else None


def _limits(memory_mb: int):
    def apply():
        import resource

        resource.setrlimit(resource.RLIMIT_AS, (memory_mb << 20, memory_mb << 20))
        resource.setrlimit(resource.RLIMIT_NPROC, (64, 64)) if hasattr(resource, "RLIMIT_NPROC") else None
        os.setsid()
    return apply


def run_program(source: str, stdin: str, timeout_s: float = 10.0, memory_mb: int = 1024) -> tuple[int, str]:
    """``source`` as a Python program in a child process of its own session, with an address-space limit, an empty
    environment and a scratch working directory; returns (exit code, stdout). A run past ``timeout_s`` is killed."""
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "main.py")
        with open(path, "w") as f:
            f.write(source)
        try:
            r = subprocess.run([sys.executable, "-I", "-S", path], input=stdin, capture_output=True, text=True, timeout=timeout_s, cwd=d,
                               env={"PATH": "/usr/bin:/bin"}, preexec_fn=_limits(memory_mb))
            return r.returncode, r.stdout
        except subprocess.TimeoutExpired:
            return -9, ""


def code_stdin(completion: str, item: dict) -> float:
    src = last_code_block(answer_part(completion))
    if src is None:
        return 0.0
    for t in item["tests"]:
        rc, out = run_program(src, t["input"], float(item.get("timeout_s", 10.0)))
        if rc != 0 or out.split() != str(t["output"]).split():
            return 0.0
    return 1.0


def exact_last_line(completion: str, item: dict) -> float:
    lines = [l.strip() for l in answer_part(completion).splitlines() if l.strip()]
    return float(bool(lines) and lines[-1] == str(item["answer"]).strip())


KINDS: dict[str, Callable[[str, dict], float]] = {
    "math_boxed": math_boxed, "multiple_choice": multiple_choice, "instruction_following": instruction_following,
    "code_stdin": code_stdin, "exact_last_line": exact_last_line,
}
