"""The general-capability protocol on CPU: scorers on hand-made completions, a run against a replica whose completions are
scripted, reuse and invalidation of finished samples, the comparison table, the router process's balancing."""

import json
import os

import pytest

from pear_b200.config.loader import compose
from pear_b200.eval import scorers
from pear_b200.eval.general import (BenchmarkRun, LeastInFlightRouter, compare_runs, dataset_status, identity, load_samples,
                                    paired_bootstrap)
from pear_b200.rollout.engine import FinishReason
from pear_b200.utils.tokenizer import ByteTokenizer


def test_math_and_choice_scorers():
    assert scorers.math_boxed("<think>maybe \\boxed{7}</think> so the answer is \\boxed{204}.", {"answer": "204"}) == 1.0
    assert scorers.math_boxed("\\boxed{\\frac{3}{4}}", {"answer": "0.75"}) == 1.0
    assert scorers.math_boxed("\\boxed{1,234}", {"answer": "1234"}) == 1.0
    assert scorers.math_boxed("\\boxed{12}", {"answer": "13"}) == 0.0
    assert scorers.math_boxed("it is 42", {"answer": "42"}) == 1.0 and scorers.math_boxed("<think>42", {"answer": "42"}) == 0.0
    assert scorers.math_boxed("\\boxed{x^{2}+1}", {"answer": "x^{2} + 1"}) == 1.0
    assert scorers.multiple_choice("Reasoning... ANSWER: C", {"answer": "C"}) == 1.0
    assert scorers.multiple_choice("The answer is (b).", {"answer": "B"}) == 1.0
    assert scorers.multiple_choice("A is tempting but I pick D", {"answer": "A"}) == 0.0
    assert scorers.multiple_choice("Answer: J", {"answer": "J", "num_options": 4}) == 0.0  # J is not an option of a 4-way item


def test_instruction_and_code_scorers():
    item = {"id": "x", "instructions": [{"id": "length:words", "args": {"relation": "at most", "n": 6}}, {"id": "case:lower"},
                                        {"id": "keywords:include", "args": {"keywords": ["pear"]}}]}
    assert scorers.instruction_following("a ripe pear falls", item) == 1.0
    assert scorers.instruction_following("A ripe pear falls", item) == 0.0
    assert scorers.instruction_following("A ripe pear falls", {**item, "strict": False}) == pytest.approx(2 / 3)
    assert scorers.instruction_following('```json\n{"a": [1, 2]}\n```', {"instructions": [{"id": "format:json"}]}) == 1.0
    assert scorers.instruction_following("* one\n* two\n", {"instructions": [{"id": "format:bullets", "args": {"n": 2}}]}) == 1.0
    with pytest.raises(ValueError, match="unknown instruction"):
        scorers.instruction_following("x", {"instructions": [{"id": "nope"}]})
    prog = "Here:\n```python\nimport sys\na, b = map(int, sys.stdin.read().split())\nprint(a + b)\n```"
    tests = [{"input": "1 2\n", "output": "3"}, {"input": "10 -4\n", "output": "6\n"}]
    assert scorers.code_stdin(prog, {"tests": tests}) == 1.0
    assert scorers.code_stdin(prog.replace("a + b", "a - b"), {"tests": tests}) == 0.0
    assert scorers.code_stdin("```python\nwhile True: pass\n```", {"tests": tests[:1], "timeout_s": 0.5}) == 0.0  # killed at its limit
    assert scorers.code_stdin("no code", {"tests": tests}) == 0.0


class _Scripted:
    """A replica whose completion for a prompt is looked up by the item text it contains."""

    def __init__(self, answers):
        self.tok, self.answers, self.calls = ByteTokenizer(), answers, 0

    def generate(self, prompt, params):
        self.calls += 1
        text = self.tok.decode(prompt, skip_special=True)
        out = next(v for k, v in self.answers.items() if k in text)

        class R:
            output = self.tok.encode(out)
            finish = FinishReason.STOP

        return R()

    def close(self):
        pass


def _protocol(tmp_path):
    ds = tmp_path / "data"
    ds.mkdir()
    (ds / "m.jsonl").write_text("\n".join(json.dumps(d) for d in [{"id": "q1", "prompt": "what is 6*7", "answer": "42"},
                                                                  {"id": "q2", "prompt": "what is 2^10", "answer": "1024"}]) + "\n")
    (ds / "c.jsonl").write_text(json.dumps({"id": "c1", "prompt": "pick the fruit", "answer": "B", "num_options": 4}) + "\n")
    cfg = compose("general", ["benchmarks={m: {file: m.jsonl, kind: math_boxed, repeats: 2, max_tokens: 64}, "
                              "c: {file: c.jsonl, kind: multiple_choice, repeats: 1, max_tokens: 64}, gone: {file: gone.jsonl, kind: math_boxed, repeats: 1, max_tokens: 8, source: elsewhere}}",
                              "concurrency=4", "bootstrap.samples=200"])
    return cfg, str(ds)


def test_run_reuses_finished_samples_and_invalidates_on_a_protocol_change(tmp_path):
    cfg, ds = _protocol(tmp_path)
    st = dataset_status(cfg, ds)
    assert st["m"] == {"present": True, "items": 2, "kind": "math_boxed"} and not st["gone"]["present"] and st["gone"]["source"] == "elsewhere"
    good = _Scripted({"6*7": "\\boxed{42}", "2^10": "so \\boxed{1000}", "fruit": "ANSWER: B"})
    out = str(tmp_path / "run_a")
    rep = BenchmarkRun(cfg, LeastInFlightRouter([good]), ByteTokenizer(), "model-a", out, ds, only=["m", "c"]).run()
    assert rep["m"]["status"] == "ok" and rep["m"]["mean"] == 0.5 and rep["c"]["mean"] == 1.0 and good.calls == 5
    assert load_samples(out, "m") == {"q1": [1.0, 1.0], "q2": [0.0, 0.0]}
    # a rerun on the same OUT generates nothing; a torn last line only costs that sample
    BenchmarkRun(cfg, LeastInFlightRouter([good]), ByteTokenizer(), "model-a", out, ds, only=["m", "c"]).run()
    assert good.calls == 5
    with open(os.path.join(out, "m", "samples.jsonl"), "r+") as f:
        lines = f.readlines()
        f.seek(0)
        f.truncate()
        f.writelines(lines[:-1] + [lines[-1][: len(lines[-1]) // 2]])
    rep = BenchmarkRun(cfg, LeastInFlightRouter([good]), ByteTokenizer(), "model-a", out, ds, only=["m"]).run()
    assert good.calls == 6 and rep["m"]["reused"] == 3
    # another sampling protocol: the old samples are set aside, everything runs again
    cfg2 = compose("general", ["sampling.temperature=0.6", "concurrency=4", "benchmarks={m: {file: m.jsonl, kind: math_boxed, repeats: 2, max_tokens: 64}}"])
    assert identity(dict(cfg["benchmarks"]["m"]), dict(cfg["sampling"]), "model-a") != identity(dict(cfg2["benchmarks"]["m"]), dict(cfg2["sampling"]), "model-a")
    BenchmarkRun(cfg2, LeastInFlightRouter([good]), ByteTokenizer(), "model-a", out, ds).run()
    assert good.calls == 10 and any(n.endswith(".stale.jsonl") for n in os.listdir(os.path.join(out, "m")))
    # a missing dataset fails its benchmark only, and the command at the end
    with pytest.raises(SystemExit, match="1 of 2 benchmarks failed: gone"):
        BenchmarkRun(cfg, LeastInFlightRouter([good]), ByteTokenizer(), "model-a", str(tmp_path / "run_c"), ds, only=["c", "gone"]).run()
    assert load_samples(str(tmp_path / "run_c"), "c") == {"c1": [1.0]}


def test_compare_table(tmp_path):
    cfg, ds = _protocol(tmp_path)
    a = _Scripted({"6*7": "\\boxed{41}", "2^10": "\\boxed{1000}", "fruit": "ANSWER: B"})
    b = _Scripted({"6*7": "\\boxed{42}", "2^10": "\\boxed{1024}", "fruit": "ANSWER: B"})
    for name, rep in (("run_a", a), ("run_b", b)):
        BenchmarkRun(cfg, LeastInFlightRouter([rep]), ByteTokenizer(), name, str(tmp_path / name), ds, only=["m", "c"]).run()
    lines = compare_runs(cfg, str(tmp_path / "run_a"), str(tmp_path / "run_b"), ("base", "tuned"))
    row_m = next(l for l in lines if l.startswith("m "))
    assert "+100.0" in row_m and row_m.rstrip().endswith("* 2")  # both items flipped: the interval excludes 0
    row_c = next(l for l in lines if l.startswith("c "))
    assert "+0.0" in row_c and "*" not in row_c
    assert any(l.startswith("gone") and "missing in a" in l for l in lines)
    r = paired_bootstrap({"x": [0.0, 1.0], "y": [1.0]}, {"x": [1.0], "y": [1.0], "z": [0.0]}, samples=100)
    assert r["items"] == 2 and r["mean_a"] == 0.75 and r["diff"] == 0.25


def test_router_process_balances_over_backends():
    """The proxy application against two stand-in backends: a request goes to the backend with fewer requests in flight."""
    import asyncio

    from aiohttp import web
    from aiohttp.test_utils import TestClient, TestServer

    from pear_b200.eval.general import router_app

    async def scenario():
        hits = {"a": 0, "b": 0}
        gate = asyncio.Event()

        def backend(tag):
            async def handle(request):
                hits[tag] += 1
                if request.path == "/slow":
                    await gate.wait()
                return web.json_response({"backend": tag, "echo": (await request.read()).decode()})
            app = web.Application()
            app.router.add_route("*", "/{tail:.*}", handle)
            return app

        sa, sb = TestServer(backend("a")), TestServer(backend("b"))
        await sa.start_server()
        await sb.start_server()
        client = TestClient(TestServer(router_app([str(sa.make_url("")), str(sb.make_url(""))])))
        await client.start_server()
        try:
            slow = asyncio.ensure_future(client.post("/slow", data=b"x"))  # occupies the first backend
            await asyncio.sleep(0.2)
            r = await client.post("/v1/completions", data=b"hello")
            body = await r.json()
            assert body == {"backend": "b", "echo": "hello"}
            gate.set()
            assert (await (await slow).json())["backend"] == "a" and hits == {"a": 1, "b": 1}
        finally:
            await client.close()
            await sa.close()
            await sb.close()

    asyncio.run(scenario())


def test_items_with_pictures_travel_as_rows_at_their_placeholders(tmp_path):
    """An image benchmark item: its picture files are read, resized to the tower's grid, encoded, and sent as rows at the
    image-pad positions of a prompt in which they follow the question; two pictures of different sizes take their own counts."""
    import numpy as np
    import torch
    from PIL import Image

    from pear_b200.eval.general import load_picture
    from pear_b200.loop.vision_encoder import VisionEncoder
    from pear_b200.models.vision import FamilyVisionConfig, FamilyVisionTower

    ds = tmp_path / "data"
    (ds / "img").mkdir(parents=True)
    rng = np.random.default_rng(0)
    Image.fromarray(rng.integers(0, 256, (37, 50, 3), dtype=np.uint8)).save(ds / "img" / "a.png")   # rounds to 40 x 48
    Image.fromarray(rng.integers(0, 256, (16, 16, 3), dtype=np.uint8)).save(ds / "img" / "b.png")
    assert load_picture(str(ds / "img" / "a.png"), 8).shape == (40, 48, 3) and load_picture(str(ds / "img" / "a.png"), 8, max_pixels=600).shape == (16, 24, 3)
    (ds / "v.jsonl").write_text(json.dumps({"id": "p1", "prompt": "which option?", "answer": "C", "num_options": 4, "images": ["img/a.png", "img/b.png"]}) + "\n")
    cfg = compose("general", ["benchmarks={v: {file: v.jsonl, kind: multiple_choice, repeats: 1, max_tokens: 16}}", "concurrency=2", "image_min_pixels=0"])
    tower = FamilyVisionTower(FamilyVisionConfig.tiny(out_hidden=24)).init_weights(0)  # patch 4, merge 2: sides in multiples of 8
    seen = {}

    class Replica:
        tok = ByteTokenizer()

        def generate(self, prompt, params, embeds=None, embeds_mask=None):
            seen.update(prompt=list(prompt), embeds=embeds, mask=embeds_mask)

            class R:
                output = Replica.tok.encode("ANSWER: C")
                finish = FinishReason.STOP

            return R()

    rep = BenchmarkRun(cfg, LeastInFlightRouter([Replica()]), ByteTokenizer(), "m", str(tmp_path / "run"), str(ds), vision=VisionEncoder(tower)).run()
    assert rep["v"]["mean"] == 1.0
    tok = ByteTokenizer()
    n_a, n_b = tower.tokens_per_image(40, 48), tower.tokens_per_image(16, 16)
    pads = [i for i, t in enumerate(seen["prompt"]) if t == tok.image_pad_id]
    assert len(pads) == n_a + n_b == 30 + 4 and seen["mask"].nonzero().flatten().tolist() == pads and seen["embeds"].shape == (len(seen["prompt"]), 24)
    with torch.no_grad():
        want = tower([torch.from_numpy(load_picture(str(ds / "img" / "b.png"), 8)).permute(2, 0, 1).float() / 127.5 - 1.0])[0]
    assert torch.allclose(seen["embeds"][pads[n_a:]], want, atol=1e-5)
    text = tok.decode(seen["prompt"])
    assert text.index("which option?") < text.index("<|vision_start|>")
    with pytest.raises(SystemExit, match="1 of 1 benchmarks failed"):  # pictures without a tower: the benchmark fails by name
        BenchmarkRun(cfg, LeastInFlightRouter([Replica()]), ByteTokenizer(), "m", str(tmp_path / "run2"), str(ds)).run()
