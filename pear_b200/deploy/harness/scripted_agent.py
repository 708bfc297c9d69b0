"""A minimal agent that speaks both of the harness's protocols: the line protocol on its pipes and the Messages form to
``ANTHROPIC_BASE_URL``. It is the harness's default agent command and what its tests drive; a real agent CLI takes its place in
a deployment. Per user message it asks the model once and reports the answer; when the model server answers "prompt is too
long" it compacts: it asks for a summary of its history (the instruction opens with the marker agents of this protocol use),
replaces the history by the summary plus the current message, notes the boundary and asks again.

Options (environment): ``SCRIPTED_AGENT_STREAM=1`` asks for event streams; ``SCRIPTED_AGENT_MAX_TOKENS`` (default 64).
"""

from __future__ import annotations

import json
import os
import sys
import urllib.error
import urllib.request

MARKER = "CRITICAL: Respond with TEXT ONLY."


def post(url: str, body: dict):
    """(status, parsed body or event list)."""
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"content-type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=600) as r:
            raw, status, ctype = r.read(), r.status, r.headers.get("content-type", "")
    except urllib.error.HTTPError as e:
        raw, status, ctype = e.read(), e.code, e.headers.get("content-type", "")
    if "event-stream" in ctype:
        events = [json.loads(line[5:]) for frame in raw.split(b"\n\n") for line in frame.split(b"\n") if line.startswith(b"data:")]
        text = "".join((e.get("delta") or {}).get("text", "") for e in events if e.get("type") == "content_block_delta")
        stop = next(((e.get("delta") or {}).get("stop_reason") for e in events if e.get("type") == "message_delta"), None)
        return status, {"content": [{"type": "text", "text": text}], "stop_reason": stop}
    try:
        return status, json.loads(raw)
    except ValueError:
        return status, {"error": {"message": raw.decode(errors="replace")}}


def text_of(answer: dict) -> str:
    return "".join(b.get("text", "") for b in answer.get("content", []) if b.get("type") == "text")


def emit(obj: dict) -> None:
    sys.stdout.write(json.dumps(obj) + "\n")
    sys.stdout.flush()


def main() -> None:
    base = os.environ["ANTHROPIC_BASE_URL"].rstrip("/")
    stream = os.environ.get("SCRIPTED_AGENT_STREAM") == "1"
    max_tokens = int(os.environ.get("SCRIPTED_AGENT_MAX_TOKENS", "64"))
    model = os.environ.get("SCRIPTED_AGENT_MODEL", "agent-default")
    history: list[dict] = []
    emit({"type": "system", "subtype": "init", "data": {"base_url": base}})
    for line in sys.stdin:
        try:
            msg = json.loads(line)
        except ValueError:
            continue
        if msg.get("type") != "user":
            continue  # control requests: a request in flight ends when the proxy drops it
        user = msg["message"]
        history.append(user)
        for attempt in range(3):
            body = {"model": model, "system": "You are a scripted agent.", "messages": history, "max_tokens": max_tokens, "stream": stream}
            try:
                status, answer = post(base + "/v1/messages", body)
            except OSError as e:  # the proxy dropped the request (an interrupt) or is gone
                emit({"type": "result", "subtype": "error", "is_error": True, "result": f"request failed: {e}"})
                break
            if status == 200:
                history.append({"role": "assistant", "content": answer.get("content", [])})
                emit({"type": "assistant", "message": {"role": "assistant", "content": answer.get("content", [])}})
                emit({"type": "result", "subtype": "success", "is_error": False, "result": text_of(answer)})
                break
            message = (answer.get("error") or {}).get("message", "")
            if status == 400 and "prompt is too long" in message and len(history) > 1:
                instruction = {"type": "text", "text": MARKER + " Summarise the conversation so far."}
                last = history[-1]
                blocks = last["content"] if isinstance(last["content"], list) else [{"type": "text", "text": last["content"]}]
                asked = history[:-1] + [{"role": "user", "content": [*blocks, instruction]}]
                s_status, summary = post(base + "/v1/messages", {"model": model, "messages": asked, "max_tokens": max_tokens, "stream": stream})
                if s_status != 200:
                    continue  # a failed compaction is asked again
                head = {"type": "text", "text": "Summary of the conversation so far:\n" + text_of(summary)}
                history = [{"role": "user", "content": [head, *blocks]}]
                emit({"type": "system", "subtype": "compact_boundary", "data": {"trigger": "auto"}})
                continue
            emit({"type": "result", "subtype": "error", "is_error": True, "result": f"{status}: {message}"})
            break
        else:
            emit({"type": "result", "subtype": "error", "is_error": True, "result": "no answer within three attempts"})


if __name__ == "__main__":
    main()
