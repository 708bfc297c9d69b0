"""The agent harness (session service + upstream proxy) with the scripted agent as its agent process, against a scripted model
server and against a real (tiny, CPU) rollout replica's Messages routes."""

import asyncio
import base64
import io
import json
import os
import sys
import uuid

import pytest

aiohttp = pytest.importorskip("aiohttp")
from aiohttp import web  # noqa: E402

from pear_b200.deploy.harness.proxy import EngineMetrics, RequestAudit, UpstreamProxy  # noqa: E402
from pear_b200.deploy.harness.service import SessionService  # noqa: E402

AGENT = [sys.executable, "-m", "pear_b200.deploy.harness.scripted_agent"]
ENV = {"PATH": os.environ.get("PATH", ""), "PYTHONPATH": os.path.dirname(os.path.dirname(os.path.abspath(__file__)))}


def jpeg(color=(200, 30, 30), size=(32, 24)) -> str:
    from PIL import Image

    buf = io.BytesIO()
    Image.new("RGB", size, color).save(buf, "JPEG")
    return base64.b64encode(buf.getvalue()).decode()


class ScriptedUpstream:
    """A model server with the three Messages routes whose answers the test scripts."""

    def __init__(self, limit=2000):
        self.limit, self.seen, self.answers, self.delay_on, self.dropped, self.answer_fn = limit, [], [], None, 0, None

    @staticmethod
    def tokens(body) -> int:
        n = len(str(body.get("system") or "")) // 4
        for m in body.get("messages", []):
            for b in UpstreamProxy.blocks(m.get("content")):
                n += len(b.get("text", "")) // 4 if b.get("type") == "text" else 100
        return n

    async def start(self):
        app = web.Application(client_max_size=1 << 28)
        app.router.add_get("/v1/models", lambda r: web.json_response({"data": [{"id": "m", "max_model_len": self.limit}]}))
        app.router.add_get("/health", lambda r: web.json_response({"ok": True}))
        app.router.add_get("/metrics", lambda r: web.Response(text='# TYPE pear_num_running gauge\npear_num_running{replica="m"} 1.0\npear_other 3\n'))
        app.router.add_post("/v1/messages/count_tokens", self.count)
        app.router.add_post("/v1/messages", self.messages)
        self.runner = web.AppRunner(app, handler_cancellation=True)
        await self.runner.setup()
        site = web.TCPSite(self.runner, "127.0.0.1", 0)
        await site.start()
        self.url = f"http://127.0.0.1:{self.runner.addresses[0][1]}"
        return self

    async def count(self, request):
        return web.json_response({"input_tokens": self.tokens(await request.json())})

    async def messages(self, request):
        body = await request.json()
        self.seen.append(body)
        flat = json.dumps(body["messages"])
        if self.delay_on and self.delay_on in flat:
            try:
                await asyncio.sleep(30)
            except asyncio.CancelledError:
                self.dropped += 1
                raise
        if self.answer_fn is not None:
            text, stop = self.answer_fn(body), "end_turn"
        elif self.answers:
            text, stop = self.answers.pop(0)
        elif "about to be replaced by your summary" in flat:
            text, stop = "<summary>the robot moved the cup</summary>", "end_turn"
        else:
            text, stop = f"answer {len(self.seen)}", "end_turn"
        usage = {"input_tokens": self.tokens(body) - 5, "cache_read_input_tokens": 5, "cache_creation_input_tokens": 0, "output_tokens": len(text) // 4 + 1}
        msg = {"id": "msg_1", "type": "message", "role": "assistant", "content": [{"type": "text", "text": text}], "stop_reason": stop, "usage": usage}
        if not body.get("stream"):
            return web.json_response(msg)
        from pear_b200.rollout.messages_api import MessagesFrontend

        resp = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
        await resp.prepare(request)
        for frame in MessagesFrontend.events(msg):
            await resp.write(frame)
        await resp.write_eof()
        return resp


class Harness:
    def __init__(self, upstream_url, tmp_path, env=None, command=AGENT, **kw):
        self.svc = SessionService(upstream_url, "m", command, audit_dir=str(tmp_path / "audit"), agent_env={**ENV, **(env or {})}, **kw)

    async def __aenter__(self):
        self.runner = web.AppRunner(self.svc.app(), handler_cancellation=True)
        await self.runner.setup()
        site = web.TCPSite(self.runner, "127.0.0.1", 0)
        await site.start()
        self.url = f"http://127.0.0.1:{self.runner.addresses[0][1]}"
        self.http = aiohttp.ClientSession()
        return self

    async def __aexit__(self, *exc):
        await self.http.close()
        await self.runner.cleanup()

    async def open(self, system="You drive a robot arm.", model="m"):
        sid = str(uuid.uuid4())
        async with self.http.post(self.url + "/sessions", json={"session_id": sid, "model": model, "system": system}) as r:
            return sid, r.status

    async def turn(self, sid, text, images=(), references=(), turn_id=None):
        body = {"turn_id": turn_id or str(uuid.uuid4()), "text": text, "images": list(images), "reference_images": list(references)}
        async with self.http.post(f"{self.url}/sessions/{sid}/turns", json=body) as r:
            if r.status != 200:
                return r.status, await r.text()
            return 200, [json.loads(line) async for line in r.content if line.strip()]


def _short_instruction(tmp_path) -> str:
    """A deployment's own compaction instruction, short enough for the tests' small contexts."""
    path = tmp_path / "summary.md"
    path.write_text("CRITICAL: Respond with TEXT ONLY. The conversation is about to be replaced by your summary: <summary>...</summary>")
    return str(path)


def run(coro):
    return asyncio.run(asyncio.wait_for(coro, 120))


@pytest.mark.parametrize("stream", ["0", "1"])
def test_a_turn_reaches_the_model_server_rewritten_sized_and_recorded(tmp_path, stream):
    async def go():
        up = await ScriptedUpstream().start()
        async with Harness(up.url, tmp_path, env={"SCRIPTED_AGENT_STREAM": stream}, chat_template_kwargs={"enable_thinking": False}) as h:
            async with h.http.get(h.url + "/health") as r:
                health = await r.json()
            assert health["status"] == "ok" and health["context_limit"] == 2000 and health["capabilities"]["reference_images"]
            sid, status = await h.open()
            assert status == 200
            cam, ref = jpeg(), jpeg((10, 200, 10))
            status, events = await h.turn(sid, "Pick up the cup.", images=[{"role": "wrist", "data": cam}], references=[{"data": ref}])
            assert status == 200 and events[-1]["type"] == "result" and events[-1]["text"] == "answer 1" and not events[-1]["is_error"]
            kinds = [e["type"] for e in events]
            assert "text" in kinds and "usage" in kinds and kinds.index("text") < kinds.index("result")
            usage = events[-1]["usage"]
            assert usage["requests"] == 1 and usage["cached_tokens"] == 5 and usage["context_tokens"] == up.tokens(up.seen[0]) and usage["is_final"]
            assert usage["engine"] == {"num_running": 1.0}  # (only the kept gauges of the model server's /metrics)
            sent = up.seen[0]
            assert sent["system"] == "You drive a robot arm." and sent["metadata"]["user_id"] == sid and sent["chat_template_kwargs"] == {"enable_thinking": False}
            blocks = sent["messages"][0]["content"]
            assert [b["type"] for b in blocks] == ["image", "text", "text", "image"]  # the task's picture, the text, the label, the camera
            assert blocks[0]["source"]["data"] == ref and blocks[2]["text"] == "[wrist]" and blocks[3]["source"]["data"] == cam
            assert sent["max_tokens"] == 2000 - up.tokens(sent) and bool(sent.get("stream")) == (stream == "1")
            assert "temperature" not in sent  # sampling is the server's
            # the second turn: the first turn's picture is put back into the history the agent sends
            status, events = await h.turn(sid, "Now the plate.", images=[{"role": "wrist", "data": jpeg((1, 2, 3))}])
            assert status == 200 and events[-1]["text"] == "answer 2"
            second = up.seen[1]["messages"]
            assert len(second) == 3 and second[0]["content"][3]["source"]["data"] == cam and second[1]["role"] == "assistant"
            # the record: one line a request, pictures as digests
            lines = [json.loads(x) for x in open(tmp_path / "audit" / f"{sid}.jsonl")]
            assert [x["kind"] for x in lines] == ["main", "main"] and lines[0]["outcome"]["status"] == 200
            assert cam not in json.dumps(lines) and "data_sha256" in json.dumps(lines[0]["upstream_request"])
            placeholder = lines[0]["agent_request"]["messages"][0]["content"][2]["text"]
            assert placeholder.startswith("[camera image ") and lines[0]["agent_request"]["system"] == "You are a scripted agent."
            async with h.http.delete(f"{h.url}/sessions/{sid}") as r:
                assert (await r.json())["closed"]
            status, _ = await h.turn(sid, "again")
            assert status == 410
        await up.runner.cleanup()

    run(go())


def test_a_full_context_is_compacted_with_the_deployments_instruction_and_without_the_last_pictures(tmp_path):
    async def go():
        up = await ScriptedUpstream(limit=480).start()
        async with Harness(up.url, tmp_path, summary_prompt=_short_instruction(tmp_path)) as h:
            sid, _ = await h.open(system="S" * 40)
            notes, results = [], []
            for i in range(4):  # each turn adds about 130 tokens (a picture counts 100): the fourth finds no room
                status, events = await h.turn(sid, f"step {i} " + "x" * 80, images=[{"role": "top", "data": jpeg((i, i, i))}])
                assert status == 200
                notes += [e for e in events if e["type"] == "note" and e.get("subtype") == "compact_boundary"]
                results.append(events[-1])
            assert len(notes) == 1 and all(not r["is_error"] for r in results) and results[-1]["usage"]["compactions"] == 1
            summaries = [b for b in up.seen if "about to be replaced by your summary" in json.dumps(b["messages"])]
            assert len(summaries) == 1
            last = summaries[0]["messages"][-1]["content"]
            assert [b["type"] for b in last] == ["text", "text"] and "CRITICAL" in last[1]["text"] and "Summarise the conversation so far" not in last[1]["text"]
            assert any(b["type"] == "image" for m in summaries[0]["messages"][:-1] for b in m["content"] if isinstance(m["content"], list))  # earlier turns keep theirs
            after = up.seen[-1]["messages"]  # the request after the compaction: the summary, then the turn with its picture
            assert len(after) == 1 and "the robot moved the cup" in after[0]["content"][0]["text"] and after[0]["content"][-1]["type"] == "image"
            kinds = [json.loads(x)["kind"] for x in open(tmp_path / "audit" / f"{sid}.jsonl")]
            assert kinds.count("summary") == 1 and kinds[-1] == "main"
            too_long = [json.loads(x) for x in open(tmp_path / "audit" / f"{sid}.jsonl") if json.loads(x)["outcome"].get("status") == 400]
            assert len(too_long) == 1
        await up.runner.cleanup()

    run(go())


def test_a_summary_without_its_closing_tag_is_asked_again_and_a_cut_answer_executes_nothing(tmp_path):
    async def go():
        up = await ScriptedUpstream(limit=360).start()
        async with Harness(up.url, tmp_path, summary_prompt=_short_instruction(tmp_path)) as h:
            sid, _ = await h.open()
            for i in range(2):
                await h.turn(sid, f"step {i} " + "x" * 80, images=[{"role": "top", "data": jpeg((i, i, i))}])
            up.answers = [("<summary>cut off", "max_tokens")]  # the first summary: no closing tag
            status, events = await h.turn(sid, "step 2 " + "x" * 80, images=[{"role": "top", "data": jpeg()}])
            assert status == 200 and not events[-1]["is_error"] and events[-1]["usage"]["compactions"] == 1
            kinds = [(json.loads(x)["kind"], json.loads(x)["outcome"].get("status")) for x in open(tmp_path / "audit" / f"{sid}.jsonl")]
            assert ("summary", 500) in kinds and ("summary", 200) in kinds
            up.answers = [("half an act", "max_tokens")]
            status, events = await h.turn(sid, "go on")
            assert events[-1]["is_error"] and events[-1]["stop"] == "refused" and "cut" in events[-1]["message"]
        await up.runner.cleanup()

    run(go())


def test_requests_outside_a_turn_bad_input_and_used_ids_are_refused(tmp_path):
    async def go():
        up = await ScriptedUpstream().start()
        async with Harness(up.url, tmp_path) as h:
            sid, status = await h.open()
            assert status == 200
            async with h.http.post(f"{h.svc.proxy.url}/{sid}/v1/messages", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5}) as r:
                assert r.status == 409 and r.headers["x-should-retry"] == "false"
            assert not up.seen
            async with h.http.post(f"{h.svc.proxy.url}/{sid}/v1/messages/count_tokens", json={"messages": [{"role": "user", "content": "x" * 40}]}) as r:
                assert (await r.json())["input_tokens"] == 10 + len("You drive a robot arm.") // 4  # counted with the service's system prompt
            async with h.http.post(h.url + "/sessions", json={"session_id": sid, "model": "m", "system": "s"}) as r:
                assert r.status == 409
            async with h.http.post(h.url + "/sessions", json={"session_id": "nope", "model": "m", "system": "s"}) as r:
                assert r.status == 400
            async with h.http.post(h.url + "/sessions", json={"session_id": str(uuid.uuid4()), "model": "other", "system": "s"}) as r:
                assert r.status == 400
            status, text = await h.turn(sid, "look", images=[{"role": "top", "data": base64.b64encode(b"not a jpeg").decode()}])
            assert status == 400 and "JPEG" in text
            status, _ = await h.turn(sid, "look", images=[{"role": "top", "data": jpeg()}, {"role": "top", "data": jpeg()}])
            assert status == 400
            status, _ = await h.turn(str(uuid.uuid4()), "look")
            assert status == 410
            sid2, status = await h.open()  # a newer session replaces the one that runs; the old id is spent
            assert status == 200
            async with h.http.post(h.url + "/sessions", json={"session_id": sid, "model": "m", "system": "s"}) as r:
                assert r.status == 409
        await up.runner.cleanup()

    run(go())


def test_an_interrupt_drops_the_request_in_flight_and_a_dead_agent_loses_the_session(tmp_path):
    async def go():
        up = await ScriptedUpstream().start()
        up.delay_on = "slow one"
        async with Harness(up.url, tmp_path) as h:
            sid, _ = await h.open()
            tid = str(uuid.uuid4())
            task = asyncio.ensure_future(h.turn(sid, "slow one", turn_id=tid))
            while not up.seen:
                await asyncio.sleep(0.02)
            status, text = await h.turn(sid, "second at once")
            assert status == 409  # one turn at a time
            async with h.http.post(f"{h.url}/sessions/{sid}/turns/{tid}/interrupt") as r:
                assert (await r.json())["status"] == "stopped"
            status, events = await task
            assert events[-1]["stop"] == "interrupted" and up.dropped == 1
            up.delay_on = None
            status, events = await h.turn(sid, "fine again")  # the session goes on
            assert status == 200 and not events[-1]["is_error"]
        async with Harness(up.url, tmp_path, command=[sys.executable, "-c", "import sys; sys.stdin.readline()"]) as h:
            sid, status = await h.open()
            assert status == 200
            status, events = await h.turn(sid, "anyone there")
            assert events[-1]["stop"] == "lost" and events[-1]["is_error"]
            status, _ = await h.turn(sid, "again")
            assert status == 410
        async with Harness(up.url, tmp_path, command=["/nonexistent/agent"]) as h:
            _, status = await h.open()
            assert status == 503
        await up.runner.cleanup()

    run(go())


def test_audit_digests_and_metrics_parsing():
    d = RequestAudit.digested({"a": [{"type": "base64", "media_type": "image/jpeg", "data": "QUJD"}], "b": "keep"})
    assert d["b"] == "keep" and d["a"][0]["data_bytes"] == 4 and "data" not in d["a"][0] and len(d["a"][0]["data_sha256"]) == 64
    m = EngineMetrics.parse('# TYPE x gauge\npear_num_running{replica="r"} 2.0\npear_cache_hit_rate 0.5\nbroken line x\n')
    assert m == {"num_running": 2.0, "cache_hit_rate": 0.5}


def _tiny_server(with_vision=False):
    import torch

    from pear_b200.models.config import HybridConfig
    from pear_b200.models.hybrid import HybridForCausalLM
    from pear_b200.rollout.engine import EngineConfig
    from pear_b200.rollout.server import build_server
    from pear_b200.utils.tokenizer import ByteTokenizer

    cfg = HybridConfig.tiny()
    model = HybridForCausalLM(cfg, with_mtp=False).init_weights(3)
    srv = build_server(model, EngineConfig(num_blocks=64, block_size=16, max_num_seqs=4), name="tiny")
    vision = None
    if with_vision:
        from pear_b200.loop.vision_encoder import VisionEncoder
        from pear_b200.models.vision import VisionConfig, VisionTower

        torch.manual_seed(0)
        vision = VisionEncoder(VisionTower(VisionConfig.tiny(out_hidden=cfg.hidden_size)), "cpu")
    return srv, ByteTokenizer(), vision


def test_messages_routes_of_a_replica_count_answer_stream_and_refuse_what_does_not_fit():
    from fastapi.testclient import TestClient

    srv, tok, vision = _tiny_server(with_vision=True)
    try:
        client = TestClient(srv.http_app(tok, vision=vision))
        assert client.get("/v1/models").json()["data"][0] == {"id": "tiny", "object": "model", "max_model_len": 1024}
        body = {"model": "tiny", "system": "be brief", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0.0}
        n = client.post("/v1/messages/count_tokens", json=body).json()["input_tokens"]
        want = len(tok.render_turn("system", "be brief") + tok.render_turn("user", "hello") + tok.generation_prompt())
        assert n == want
        out = client.post("/v1/messages", json=body).json()
        assert out["type"] == "message" and out["role"] == "assistant" and out["content"][0]["type"] == "text" and out["stop_reason"] in ("end_turn", "max_tokens")
        u = out["usage"]
        assert u["input_tokens"] + u["cache_read_input_tokens"] == n and 1 <= u["output_tokens"] <= 6
        again = client.post("/v1/messages", json={**body, "metadata": {"user_id": "s1"}}).json()
        assert again["content"] == out["content"]  # greedy: the same answer
        streamed = client.post("/v1/messages", json={**body, "stream": True})
        assert streamed.headers["content-type"].startswith("text/event-stream")
        events = [json.loads(line[5:]) for line in streamed.text.splitlines() if line.startswith("data:")]
        assert [e["type"] for e in events][0] == "message_start" and events[-1]["type"] == "message_stop"
        text = "".join(e["delta"]["text"] for e in events if e["type"] == "content_block_delta")
        assert text == out["content"][0]["text"]
        # tokens go out as the engine produces them: a longer answer arrives in several deltas that add up to the whole answer
        longer = {**body, "max_tokens": 48}
        whole = client.post("/v1/messages", json=longer).json()
        events = [json.loads(line[5:]) for line in client.post("/v1/messages", json={**longer, "stream": True}).text.splitlines() if line.startswith("data:")]
        deltas = [e["delta"]["text"] for e in events if e["type"] == "content_block_delta"]
        assert len(deltas) > 1 and "".join(deltas) == whole["content"][0]["text"]
        closing = next(e for e in events if e["type"] == "message_delta")
        assert closing["delta"]["stop_reason"] == whole["stop_reason"] and closing["usage"]["output_tokens"] == whole["usage"]["output_tokens"]
        assert events[0]["message"]["usage"]["input_tokens"] + events[0]["message"]["usage"]["cache_read_input_tokens"] == n
        # a picture: placeholders are counted, rows are computed by the encoder, and the answer differs from the text-only one's prompt
        with_picture = {**body, "messages": [{"role": "user", "content": [{"type": "text", "text": "hello"},
                                                                          {"type": "image", "source": {"type": "base64", "media_type": "image/jpeg", "data": jpeg(size=(28, 28))}}]}]}
        gh, gw = vision.grid(__import__("numpy").zeros((28, 28, 3), dtype="uint8"))
        assert client.post("/v1/messages/count_tokens", json=with_picture).json()["input_tokens"] == n + gh * gw + 2
        assert client.post("/v1/messages", json=with_picture).json()["usage"]["output_tokens"] >= 1
        long = {**body, "messages": [{"role": "user", "content": "x" * 2000}]}
        r = client.post("/v1/messages", json=long)
        assert r.status_code == 400 and "prompt is too long" in r.json()["error"]["message"]
        no_vision = TestClient(srv.http_app(tok))
        assert no_vision.post("/v1/messages", json=with_picture).status_code == 400
    finally:
        srv.close()


def test_the_harness_in_front_of_a_real_replica(tmp_path):
    """The whole chain on CPU: client -> session service -> scripted agent process -> proxy -> a tiny replica's Messages routes."""
    import socket
    import threading

    import uvicorn

    srv, tok, _ = _tiny_server()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(srv.http_app(tok), host="127.0.0.1", port=port, log_level="warning"))
    thread = threading.Thread(target=server.run, daemon=True)
    thread.start()

    async def go():
        for _ in range(200):
            if server.started:
                break
            await asyncio.sleep(0.05)
        svc_kw = dict(require_summary_end=False)
        h = Harness(f"http://127.0.0.1:{port}", tmp_path, env={"SCRIPTED_AGENT_MAX_TOKENS": "8"}, **svc_kw)
        h.svc.model = "tiny"
        async with h:
            sid, status = await h.open(system="You answer in bytes.", model="tiny")
            assert status == 200
            for i in range(2):
                status, events = await h.turn(sid, f"turn {i}: say something")
                assert status == 200 and events[-1]["type"] == "result" and events[-1]["stop"] in ("end_turn", "refused")
                assert events[-1]["usage"]["requests"] == 1 and events[-1]["usage"]["output_tokens"] >= 1
            # (a random model's bytes do not survive decoding and re-encoding, so the second turn's prompt is not a token-exact
            # continuation of the first and takes nothing from the prefix cache; a trained model's text does)
            assert events[-1]["usage"]["context_limit"] == 1024 and events[-1]["usage"]["context_tokens"] > 60

    try:
        run(go())
    finally:
        server.should_exit = True
        thread.join(timeout=10)
        srv.close()


def test_deploy_server_offers_the_messages_routes_over_its_one_session_engine():
    """The deploy server (one checkpoint, one session at a time) is the model server the harness fronts in a deployment: the same
    three routes over its engine's fixed-length decode, cut at the end-of-turn token. (A stand-in engine: the real one is a GPU
    megakernel.)"""
    from types import SimpleNamespace

    from fastapi.testclient import TestClient

    from pear_b200.deploy.server import DeployServer
    from pear_b200.utils.tokenizer import ByteTokenizer

    tok = ByteTokenizer()

    class Engine:
        max_len, temperature, seed = 256, 1.0, 0

        def generate(self, prompt, max_new_tokens):
            self.prompt = prompt.tolist()
            text = tok.encode("ok then") + [tok.eos_id] + tok.encode("never read")
            return SimpleNamespace(tokens=text[:max_new_tokens])

    engine = Engine()
    client = TestClient(DeployServer(engine, tok, name="served").http_app())
    assert client.get("/v1/models").json()["data"][0] == {"id": "served", "object": "model", "max_model_len": 256} and client.get("/health").json()["ok"]
    body = {"model": "served", "system": "s", "messages": [{"role": "user", "content": "go"}], "max_tokens": 32}
    n = client.post("/v1/messages/count_tokens", json=body).json()["input_tokens"]
    out = client.post("/v1/messages", json=body).json()
    assert out["content"][0]["text"] == "ok then" and out["stop_reason"] == "end_turn" and out["usage"]["input_tokens"] == n == len(engine.prompt)
    cut = client.post("/v1/messages", json={**body, "max_tokens": 3}).json()
    assert cut["content"][0]["text"] == "ok " and cut["stop_reason"] == "max_tokens"
    assert client.post("/v1/messages", json={**body, "messages": [{"role": "user", "content": "x" * 300}]}).status_code == 400


# -- the station: robot session in front of the harness ---------------------------------------------------------------------
def _toward_target(body) -> str:
    """A scripted policy: read the state out of the last turn's text and move toward (0.7, 0.6), at most 0.2 an axis."""
    import re

    text = " ".join(b.get("text", "") for b in UpstreamProxy.blocks(body["messages"][-1]["content"]) if b.get("type") == "text")
    state = json.loads(re.findall(r"State: (\{.*?\})", text)[-1])
    dx, dy = (max(-0.2, min(0.2, t - state[k])) for t, k in ((0.7, "x"), (0.6, "y")))
    action = {"arm": {"dx": round(dx, 4), "dy": round(dy, 4), "dz": 0.0}, "gripper": {"opening": 0.5}}
    return "The target is to the right.\n```json\n" + json.dumps(action) + "\n```"


def test_action_parser_takes_only_a_whole_answer_that_ends_with_one_action_of_the_format():
    from pear_b200.deploy.station.action_parser import parse_action
    from pear_b200.deploy.station.robot import CARTESIAN

    good = {"arm": {"dx": 0.1, "dy": 0, "dz": -0.05}, "gripper": {"opening": 1}}
    fenced = lambda obj: "so:\n```json\n" + (obj if isinstance(obj, str) else json.dumps(obj)) + "\n```"  # noqa: E731
    assert parse_action(fenced(good), CARTESIAN) == good
    assert parse_action("```json\n{}\n```\nno, rather\n" + fenced(good), CARTESIAN) == good  # the last block counts
    for bad in (fenced(good) + "\nand then some", "<think>hm</think>" + fenced(good), "no action here", fenced({"arm": good["arm"]}),
                fenced({**good, "extra": {}}), fenced({"arm": {"dx": 0.1, "dy": 0}, "gripper": good["gripper"]}),
                fenced({"arm": {"dx": True, "dy": 0, "dz": 0}, "gripper": good["gripper"]}), fenced({"arm": {"dx": 0.5, "dy": 0, "dz": 0}, "gripper": good["gripper"]}),
                fenced('{"arm": {"dx": 0.1, "dx": 0.2, "dy": 0, "dz": 0}, "gripper": {"opening": 1}}'), fenced('{"arm": {"dx": NaN, "dy": 0, "dz": 0}, "gripper": {"opening": 1}}'),
                fenced("{not json")):
        with pytest.raises(ValueError):
            parse_action(bad, CARTESIAN)


def test_station_loop_executes_only_parsed_actions_records_turns_and_ends_requests_it_gives_up_on(tmp_path):
    import threading
    import time

    from pear_b200.deploy.station.agent_loop import OperatorPaused, StationAgentLoop, system_prompt
    from pear_b200.deploy.station.clients import ContextLimit, ModelClient, ModelOutput
    from pear_b200.deploy.station.robot import CARTESIAN, SimulatedArm

    class Scripted(ModelClient):
        def __init__(self):
            super().__init__("s")
            self.script, self.inputs, self.cancelled, self.closed = [], [], 0, False

        def infer(self, model_input, on_event, cancellation):
            self.inputs.append(model_input)
            item = self.script.pop(0)
            if item == "hang":
                while not cancellation.is_set():
                    time.sleep(0.01)
                raise InterruptedError("stopped")
            if isinstance(item, Exception):
                raise item
            return ModelOutput(item, 0.01, {"output_tokens": 3})

        def cancel(self):
            self.cancelled += 1

        def close(self):
            self.closed = True

    act = lambda dx, dy: "ok\n```json\n" + json.dumps({"arm": {"dx": dx, "dy": dy, "dz": 0.0}, "gripper": {"opening": 0.3}}) + "\n```"  # noqa: E731
    arm, client, events = SimulatedArm(), Scripted(), []
    loop = StationAgentLoop(arm, client, CARTESIAN, timeout_s=0.3, directory=str(tmp_path / "task"))
    assert "```json" in system_prompt("put the cup away", CARTESIAN) and '"dx": <number>' in system_prompt("x", CARTESIAN)
    on_event, never = (lambda kind, data: events.append((kind, data))), threading.Event()
    client.script = [act(0.2, 0.2), "I would rather not say", act(0.2, 0.2), act(0.2, 0.2), "hang"]
    r1 = loop.step(never, on_event)
    assert r1.status == "completed" and arm.state()["x"] == 0.4 and arm.state()["opening"] == 0.3
    r2 = loop.step(never, on_event)  # no action in the answer: nothing moves, the model is told next turn
    assert r2.status == "rejected" and arm.moves == 1 and not loop.last_turn.dispatched
    r3 = loop.step(never, on_event)
    assert r3.status == "completed" and "was not sent to the robot" in client.inputs[2].text and "ended as rejected" in client.inputs[2].text
    r4 = loop.step(never, on_event)  # x would be 0.8 + ... fine; y 0.8: still inside; one more would leave
    assert r4.status == "completed" and "The last action completed." in client.inputs[3].text
    t0 = time.time()
    r5 = loop.step(never, on_event)  # the model hangs: the request is ended after the timeout, the turn fails, the session goes on
    assert r5.status == "failed" and "did not answer within" in r5.detail and client.cancelled == 1 and time.time() - t0 < 5
    client.script = [act(0.2, 0.2)]
    arm.pos[:2] = (0.9, 0.9)
    r6 = loop.step(never, on_event)  # 0.9 + 0.2: outside the workspace: the robot itself refuses a dispatched action
    assert r6.status == "rejected" and loop.last_turn.dispatched and "workspace" in r6.detail
    # the operator's stop ends the request in flight too
    client.script = ["hang"]
    stop = threading.Event()
    threading.Timer(0.1, stop.set).start()
    with pytest.raises(OperatorPaused):
        loop.step(stop, on_event)
    assert client.cancelled == 2 and loop.previous_result.status == "stopped"
    # a conversation that cannot go on blocks the session for good
    client.script = [ContextLimit("prompt is too long: 9 tokens > 8 maximum")]
    with pytest.raises(ContextLimit):
        loop.step(never, on_event)
    with pytest.raises(ContextLimit):
        loop.step(never, on_event)
    assert len(client.inputs) == 8  # (the blocked step asked nobody)
    records = [json.loads(x) for x in open(tmp_path / "task" / "turns.jsonl")]
    assert [r["result"]["status"] for r in records] == ["completed", "rejected", "completed", "completed", "failed", "rejected", "stopped", "failed"]
    assert records[0]["action"]["arm"]["dx"] == 0.2 and records[1]["action"] is None and records[0]["usage"] == {"output_tokens": 3}
    assert len([f for f in os.listdir(tmp_path / "task") if f.endswith("_top.jpg")]) == 8
    assert [k for k, _ in events[:6]] == ["phase", "observation", "phase", "model_output", "action", "phase"]
    loop.close()
    assert client.closed


@pytest.mark.parametrize("kind", ["harness", "messages"])
def test_a_simulated_arm_reaches_its_target_through_the_whole_deployment_chain(tmp_path, kind):
    """station loop -> model client -> (session service -> agent process -> proxy ->) model server with a scripted policy."""
    import threading

    from pear_b200.deploy.station.agent_loop import StationAgentLoop, system_prompt
    from pear_b200.deploy.station.clients import HarnessClient, MessagesClient
    from pear_b200.deploy.station.robot import CARTESIAN, SimulatedArm

    ready, stop, box = threading.Event(), threading.Event(), {}

    async def serve():
        up = await ScriptedUpstream(limit=3000).start()
        up.answer_fn = _toward_target
        async with Harness(up.url, tmp_path) as h:
            box.update(up=up, upstream=up.url, service=h.url)
            ready.set()
            while not stop.is_set():
                await asyncio.sleep(0.05)
        await up.runner.cleanup()

    thread = threading.Thread(target=lambda: asyncio.run(serve()), daemon=True)
    thread.start()
    assert ready.wait(30)
    try:
        arm = SimulatedArm()
        prompt = system_prompt("Move the gripper over the green target.", CARTESIAN)
        client = HarnessClient(box["service"], "m", prompt) if kind == "harness" else MessagesClient(box["upstream"], "m", prompt)
        assert client.check()["status"] == "ok"
        loop = StationAgentLoop(arm, client, CARTESIAN, timeout_s=60, directory=str(tmp_path / "task"), reference_images=(arm.observe().cameras["top"],))
        never = threading.Event()
        from pear_b200.deploy.station.records import TaskRecords

        records = TaskRecords(str(tmp_path / "task"))
        for _ in range(6):
            if arm.distance() < 0.02:
                break
            assert loop.step(never, records.on_event).status == "completed"
        events = [json.loads(x) for x in open(tmp_path / "task" / "events.jsonl")]
        assert [e["type"] for e in events].count("action") == 3 and all("monotonic" in e for e in events)
        usage = json.load(open(tmp_path / "task" / "context_usage.json"))
        assert usage["turns"] == 3 and usage["output_tokens"] > 0 and len(usage["per_turn"]) == 3
        if kind == "harness":  # the service reports the context against the model's limit
            assert usage["context_limit"] == 3000 and 0 < usage["context_fraction"] < 1 and usage["compactions"] == 0
        assert arm.distance() < 0.02 and arm.moves == 3  # 0.5 in x at 0.2 a turn
        seen = box["up"].seen
        assert seen[0]["system"] == prompt and seen[0]["messages"][0]["content"][0]["type"] == "image"  # the task's reference picture leads
        assert sum(b["type"] == "image" for b in UpstreamProxy.blocks(seen[-1]["messages"][-1]["content"])) == 1  # the turn's camera
        assert len(seen[-1]["messages"]) == 5  # the conversation so far: three user turns, two answers
        loop.close()
    finally:
        stop.set()
        thread.join(timeout=20)


def test_messages_client_against_a_real_replica_says_when_an_answer_is_cut_and_when_the_context_is_full():
    import threading

    import numpy as np
    from fastapi.testclient import TestClient

    from pear_b200.deploy.station.clients import ContextLimit, MessagesClient, ModelInput

    srv, tok, vision = _tiny_server(with_vision=True)
    try:
        http = TestClient(srv.http_app(tok, vision=vision))
        client = MessagesClient("", "tiny", "You move an arm.", max_tokens=4, session=http)
        assert client.check()["status"] == "ok" and client.check()["context_limit"] == 1024
        assert MessagesClient("", "other", "s", session=http).check()["status"] == "offline"
        frame = np.zeros((28, 28, 3), dtype=np.uint8)
        never = threading.Event()
        with pytest.raises(ValueError, match="cut"):  # a random model does not end its turn within four tokens
            client.infer(ModelInput("Turn 1.", {"top": frame}, (frame,)), lambda k, d: None, never)
        assert client.history == []  # a refused answer is not part of the conversation
        with pytest.raises(ContextLimit, match="prompt is too long"):
            client.infer(ModelInput("x" * 1200, {}, ()), lambda k, d: None, never)
        stop = threading.Event()
        stop.set()
        with pytest.raises(InterruptedError):
            client.infer(ModelInput("Turn 2.", {}, ()), lambda k, d: None, stop)
        client.close()
    finally:
        srv.close()
