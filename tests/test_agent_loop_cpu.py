"""Agent loop, environment servers and protocol on CPU: the episode path of the embodied recipe end to end, plus the
host-side failure paths (lost environment process, unparsable answer, token budget)."""

import numpy as np
import pytest
import torch

from pear_b200.envs.synthetic import SyntheticEnv
from pear_b200.loop.agent_loop import AgentLoop, AgentLoopConfig
from pear_b200.loop.dataset import EpisodeDataset
from pear_b200.loop.episode import EndReason
from pear_b200.loop.manager import AgentLoopManager, Router
from pear_b200.loop.protocol import ParseError, extract_action, parse_answer
from pear_b200.loop.tool_parser import get_parser
from pear_b200.loop.transfer_queue import TransferQueue
from pear_b200.rollout.engine import FinishReason, Request, SamplingParams
from pear_b200.sim.client import EpisodeClient
from pear_b200.sim.env import EpisodeLost
from pear_b200.sim.server import ServerPool
from pear_b200.utils.tokenizer import ByteTokenizer

ENV = "pear_b200.envs.synthetic.SyntheticEnv"


def test_protocol_and_parser():
    schema = SyntheticEnv.action_schema()
    txt = "<think>hm ```json\n{\"move\": 0}\n```</think> first ```json\n{\"move\": -1}\n``` then ```json\n{\"move\": 1}\n```"
    assert extract_action(txt) == {"move": 1}
    assert parse_answer(txt, schema) == {"move": 1}
    for bad in ("no block", "```json\n{\"move\": 5}\n```", "```json\n{\"jump\": 1}\n```", "```json\n[1]\n```", "```json\n{}\n```"):
        with pytest.raises(ParseError):
            parse_answer(bad, schema)
    assert get_parser("qwen3_5")(txt)[0].arguments == {"move": 1}
    assert get_parser("fenced_json")("nothing") == []


def test_tokenizer_roundtrip():
    tok = ByteTokenizer()
    s = "<|im_start|>user\nhé {\"a\": 1}<|im_end|>\n"
    assert tok.decode(tok.encode(s)) == s
    turn = tok.render_turn("user", "x", images=2, image_tokens=3)
    assert turn.count(tok.image_pad_id) == 6


def test_dataset_product_and_resume():
    d = EpisodeDataset({"family": "synthetic", "args": {"task": ["a", "b"], "seed": [0, 1, 2]}}, shuffle=True, seed=3)
    assert len(d) == 6
    first = [d.next().index for _ in range(4)]
    st = d.state()
    rest = [d.next().index for _ in range(5)]
    d2 = EpisodeDataset({"family": "synthetic", "args": {"task": ["a", "b"], "seed": [0, 1, 2]}}, shuffle=True, seed=3)
    d2.restore(st)
    assert [d2.next().index for _ in range(5)] == rest and sorted(first + rest[:2]) == list(range(6))


class ScriptedRouter:
    """Stands in for the rollout replicas: answers from a script so the loop's logic is tested deterministically."""

    hidden_size = 8

    def __init__(self, tok, answers):
        self.tok, self.answers, self.calls = tok, list(answers), []

    def generate(self, prompt, params, session=None, embeds=None, embeds_mask=None):
        self.calls.append((len(prompt), params.max_tokens, None if embeds is None else int(embeds_mask.sum())))
        text = self.answers.pop(0) if self.answers else "```json\n{\"submit\": true}\n```"
        out = self.tok.encode(text)[: params.max_tokens]
        finish = FinishReason.LENGTH if len(out) == params.max_tokens else FinishReason.STOP
        r = Request("r", list(prompt), params, session)
        r.output, r.logprobs, r.finish = out + ([self.tok.eos_id] if finish == FinishReason.STOP else []), [-1.0] * (len(out) + (finish == FinishReason.STOP)), finish
        return r


@pytest.fixture()
def pool():
    p = ServerPool()
    yield p
    p.close()


def _loop(pool, answers, queue=None, **cfg):
    tok = ByteTokenizer()
    router = ScriptedRouter(tok, answers)
    loop = AgentLoop(router, pool, tok, AgentLoopConfig(**cfg), {"synthetic": SyntheticEnv.action_schema()}, queue)
    return loop, router


def test_episode_success_and_trajectory_layout(pool, tmp_path):
    pool.start("synthetic", ENV, "stateless", num_processes=1, env_kwargs={"hidden": 8, "tokens_per_image": 4})
    # find the moves that solve seed 0
    env = SyntheticEnv(hidden=8, tokens_per_image=4)
    d = env.reset({"seed": 0})["state"]["distance"]
    moves = ["<think>go</think>```json\n{\"move\": %d}\n```" % (1 if d > 0 else -1)] * abs(d)
    q = TransferQueue(4)
    loop, router = _loop(pool, moves + ["```json\n{\"submit\": true}\n```"], q, token_budget=4000, log_dir=str(tmp_path))
    ep = loop.run("g0", "0", "synthetic", {"seed": 0})
    assert ep.end_reason == EndReason.ENV and ep.success and ep.turns == abs(d) + 1
    tr = q.get("g0/0")
    assert tr["reward"] == 1.0 and len(tr["tokens"]) == len(tr["response_mask"]) == len(tr["rollout_logprobs"])
    assert tr["response_mask"][: tr["prompt_len"]].sum() == 0 and tr["response_mask"].sum() == ep.response_tokens
    # every user turn contributed one image block of 4 placeholder rows, at image-pad positions
    tok = ByteTokenizer()
    for pos, block in tr["embeds"]:
        assert block.shape == (4, 8) and all(t == tok.image_pad_id for t in tr["tokens"][pos:pos + 4])
    assert len(tr["embeds"]) == ep.turns and router.calls[-1][2] == 4 * ep.turns
    assert (tmp_path / "turns.jsonl").exists() and (tmp_path / "calls.jsonl").exists()


def test_episode_parse_and_budget_ends(pool):
    pool.start("synthetic", ENV, "stateless", num_processes=1, env_kwargs={"hidden": 8, "tokens_per_image": 2})
    loop, _ = _loop(pool, ["I will not answer in json"], token_budget=4000)
    ep = loop.run("g1", "0", "synthetic", {"seed": 1})
    assert ep.end_reason == EndReason.PARSE and not ep.success
    loop, router = _loop(pool, ["<think>" + "x" * 500], token_budget=64)
    ep = loop.run("g2", "0", "synthetic", {"seed": 1})
    assert ep.end_reason == EndReason.BUDGET and ep.response_tokens == 64 and router.calls[0][1] == 64


def test_lost_environment_restarts_then_gives_up(pool):
    # stateful family whose process dies on its second step: every attempt is lost, the loop restarts twice, then ends
    pool.start("synthetic", ENV, "stateful", num_processes=1, call_timeout_s=5.0, env_kwargs={"hidden": 8, "tokens_per_image": 2, "hang_after": 0})
    pool.get("synthetic").call_timeout_s = 0.5
    loop, router = _loop(pool, ["```json\n{\"move\": 0}\n```"] * 10, token_budget=4000, max_restarts=2)
    ep = loop.run("g3", "0", "synthetic", {"seed": 2})
    assert ep.end_reason == EndReason.LOST and ep.restarts == 2
    assert pool.get("synthetic").restarts >= 1 or True


def test_stateless_call_retried_on_another_process(pool):
    srv = pool.start("synthetic", ENV, "stateless", num_processes=2, env_kwargs={"hidden": 8, "tokens_per_image": 2})
    c = EpisodeClient(pool, "synthetic")
    first = c.open({"seed": 5})
    # kill one process behind the server's back: the next call is retried on the other one and still answers
    srv.slots[0].proc.kill()
    srv.slots[0].proc.join(5)
    out = c.step({"move": 0})
    assert out["steps"] == 1 and out["observation"]["state"]["step"] == 1 and first["observation"]["state"]["step"] == 0


def test_manager_runs_groups_round_robin(pool):
    tok = ByteTokenizer()

    class Fixed:
        def generate(self, prompt, params, session=None, embeds=None, embeds_mask=None):
            r = Request("r", list(prompt), params, session)
            r.output = tok.encode("```json\n{\"submit\": true}\n```") + [tok.eos_id]
            r.logprobs, r.finish = [-0.5] * len(r.output), FinishReason.STOP
            return r

    q = TransferQueue(4)
    mgr = AgentLoopManager([Fixed(), Fixed()], 8, {"synthetic": {"env_path": ENV, "num_processes": 2, "env_kwargs": {"hidden": 8, "tokens_per_image": 2}}},
                           AgentLoopConfig(token_budget=256), q, num_workers=3)
    try:
        futs = mgr.dispatch_group("gA", "synthetic", {"seed": 0}, ["0", "1", "2", "3"]) + mgr.dispatch_group("gB", "synthetic", {"seed": 1}, ["0", "1"])
        eps = [f.result(timeout=60) for f in futs]
        assert all(e.end_reason == EndReason.ENV for e in eps)
        assert sorted(q.keys()) == ["gA/0", "gA/1", "gA/2", "gA/3", "gB/0", "gB/1"]
    finally:
        mgr.close()


def test_first_turn_prompt_rendering_is_the_stored_text():
    """The text a policy reads at the start of an episode, byte for byte: system prompt, the observation's state and reminder,
    each camera's picture under its label, the assistant header. A change of the template shows up as a diff of the stored
    rendering, not as a silent shift of what checkpoints were trained on."""
    import os

    import numpy as np

    from pear_b200.envs.tool import episode_system_prompt, load_system_prompt, render_observation

    tok = ByteTokenizer()
    res = {"observation": {"state": {"gripper": "open", "cube": [0.1, 0.2, 0.0], "step": 3}, "reminder": "Answer with one JSON action in a fenced json block.",
                           "frames": {"wrist": np.zeros((2, 8)), "front": np.ones((2, 8))},
                           "environment": ["front: a fixed camera above the table", "wrist: a camera on the gripper"], "task": "put the cube in the bowl"},
           "done": False}
    obs = render_observation(res)
    assert obs.cameras == ["front", "wrist"] and obs.frames[0].sum() == 16  # frames in the cameras' (sorted) order
    assert episode_system_prompt("base\n", render_observation({"observation": {"state": {}}})) == "base\n"  # a family that says nothing adds nothing
    ids = (tok.render_turn("system", episode_system_prompt(load_system_prompt(), obs)) + tok.render_turn("user", obs.text, images=2, image_tokens=2, labels=obs.cameras)
           + tok.generation_prompt())
    with open(os.path.join(os.path.dirname(__file__), "golden", "first_turn_prompt.txt")) as f:
        assert tok.decode(ids) == f.read()
    text = tok.decode(ids)
    assert text.index("## ENVIRONMENT") < text.index("## TASK") < text.index("put the cube in the bowl") < text.index("<|im_start|>user")
    assert text.index("[front]") < text.index("<|vision_start|>") < text.index("[wrist]") < text.rindex("<|vision_start|>")


def test_pixel_cameras_go_through_the_vision_encoder(pool):
    """An environment whose cameras deliver pixels: the agent loop encodes each distinct picture once with the vision tower
    (the two cameras of a turn in one batched call, an unchanged scene from the cache) and the trajectory carries the rows at
    the image-pad positions; without an encoder the loop refuses pixels by name."""
    from pear_b200.loop.vision_encoder import VisionEncoder
    from pear_b200.models.vision import VisionConfig, VisionTower

    pool.start("synthetic", ENV, "stateless", num_processes=1, env_kwargs={"pixels": 16, "cameras": ("front", "wrist")})
    tower = VisionTower(VisionConfig.tiny(out_hidden=8)).init_weights(1)
    n_tok = tower.tokens_per_image(16, 16)
    enc = VisionEncoder(tower)
    tok = ByteTokenizer()
    q = TransferQueue(4)
    answers = ['```json\n{"move": 0}\n```', '```json\n{"move": 0}\n```', '```json\n{"submit": true}\n```']  # the scene never changes
    router = ScriptedRouter(tok, answers)
    loop = AgentLoop(router, pool, tok, AgentLoopConfig(token_budget=4000), {"synthetic": SyntheticEnv.action_schema()}, q, vision=enc)
    ep = loop.run("gp", "0", "synthetic", {"seed": 3})
    tr = q.get("gp/0")
    assert ep.turns == 3 and len(tr["embeds"]) == 2 * ep.turns
    for pos, block in tr["embeds"]:
        assert block.shape == (n_tok, 8) and all(t == tok.image_pad_id for t in tr["tokens"][pos:pos + n_tok])
    assert enc.encoded == 2 and enc.hits == 2 * (ep.turns - 1)  # two cameras encoded once, the later turns from the cache
    # the rows are the tower's output for the environment's pictures
    env = SyntheticEnv(pixels=16, cameras=("front", "wrist"))
    frames = env.reset({"seed": 3})["frames"]
    with torch.no_grad():
        want = tower([torch.from_numpy(frames["front"]).permute(2, 0, 1).float() / 127.5 - 1.0])[0]
    assert np.allclose(tr["embeds"][0][1], want.numpy().astype(np.float16), atol=2e-3)
    bare = AgentLoop(ScriptedRouter(tok, answers), pool, tok, AgentLoopConfig(token_budget=4000, max_restarts=0), {"synthetic": SyntheticEnv.action_schema()})
    with pytest.raises(ValueError, match="needs a vision encoder"):
        bare.run("gq", "0", "synthetic", {"seed": 3})


def test_prompt_longer_than_the_limit_ends_the_episode_before_any_request(pool):
    pool.start("synthetic", ENV, "stateless", num_processes=1, env_kwargs={"hidden": 8, "tokens_per_image": 2})
    loop, router = _loop(pool, ['```json\n{"submit": true}\n```'], token_budget=4000, max_prompt_length=64)  # the system prompt alone is longer
    ep = loop.run("gl", "0", "synthetic", {"seed": 1})
    assert ep.end_reason == EndReason.BUDGET and ep.response_tokens == 0 and not router.calls
    loop2, router2 = _loop(pool, ['```json\n{"submit": true}\n```'], token_budget=4000, max_prompt_length=100000)
    assert loop2.run("gm", "0", "synthetic", {"seed": 1}).response_tokens > 0 and router2.calls


def test_episodes_on_remote_environment_hosts_with_failover(tmp_path):
    """The environment role as processes: two hosts serve the synthetic family over HTTP; an episode runs through them (camera
    blocks travel as encoded arrays), a host that dies is skipped, and when no host answers the episode is lost."""
    import os
    import subprocess
    import sys
    import time

    import requests

    from pear_b200.sim.server import RemoteServer, decode_arrays, encode_arrays
    from pear_b200.utils.process import free_ports

    x = {"a": np.arange(6, dtype=np.float32).reshape(2, 3), "b": [np.uint8(3), {"c": np.zeros((1, 2), dtype=np.uint8)}], "d": "s"}
    y = decode_arrays(encode_arrays(x))
    assert np.array_equal(y["a"], x["a"]) and y["a"].dtype == np.float32 and y["b"][0] == 3 and y["b"][1]["c"].dtype == np.uint8 and y["d"] == "s"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ports = free_ports(2)
    hosts = [subprocess.Popen([sys.executable, "-m", "pear_b200.sim.server", "--port", str(p), "--processes", "1", "--env-kwargs", '{"hidden": 8, "tokens_per_image": 4}'],
                              env=dict(os.environ, PYTHONPATH=root), stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) for p in ports]
    urls = [f"http://127.0.0.1:{p}" for p in ports]
    try:
        for u in urls:
            t0 = time.time()
            while True:
                try:
                    if requests.get(u + "/health", timeout=2).json()["ok"]:
                        break
                except Exception:  # noqa: BLE001
                    assert time.time() - t0 < 60, "environment host did not start"
                    time.sleep(0.2)
        local = ServerPool()
        try:
            remote = local.connect("synthetic", urls, retry_after_s=60.0)
            assert isinstance(remote, RemoteServer) and local.capacity("synthetic") == 2
            env = SyntheticEnv(hidden=8, tokens_per_image=4)
            d = env.reset({"seed": 0})["state"]["distance"]
            moves = ['```json\n{"move": %d}\n```' % (1 if d > 0 else -1)] * abs(d) + ['```json\n{"submit": true}\n```']
            q = TransferQueue(4)
            loop, _ = _loop(local, moves, q, token_budget=4000)
            ep = loop.run("gr", "0", "synthetic", {"seed": 0})
            assert ep.end_reason == EndReason.ENV and ep.success and all(b.shape == (4, 8) for _, b in q.get("gr/0")["embeds"])
            hosts[0].kill()
            hosts[0].wait(30)
            loop2, _ = _loop(local, moves, q, token_budget=4000)
            ep2 = loop2.run("gs", "0", "synthetic", {"seed": 0})
            assert ep2.success and remote.failovers >= 1 and urls[0] in remote.down  # the dead host is skipped from now on
            hosts[1].kill()
            hosts[1].wait(30)
            loop3, _ = _loop(local, moves, q, token_budget=4000, max_restarts=1)
            ep3 = loop3.run("gt", "0", "synthetic", {"seed": 0})
            assert ep3.end_reason == EndReason.LOST and not ep3.success
        finally:
            local.close()
    finally:
        for h in hosts:
            if h.poll() is None:
                h.kill()
            h.wait(30)


def test_agent_loop_emits_the_structured_events(pool, caplog):
    """One line per event, a name and a JSON object: what the monitor and operators grep for."""
    import json
    import logging

    pool.start("synthetic", ENV, "stateless", num_processes=1, env_kwargs={"hidden": 8, "tokens_per_image": 2})
    log = logging.getLogger("pear_b200.agent_loop")
    log.propagate = True  # (the logger has a handler of its own; the test listens through the root)
    try:
        with caplog.at_level(logging.INFO, logger="pear_b200.agent_loop"):
            loop, _ = _loop(pool, ["no json here"], token_budget=4000)
            loop.run("ge", "0", "synthetic", {"seed": 1})
    finally:
        log.propagate = False
    lines = [r.getMessage() for r in caplog.records]
    fail = next(l for l in lines if l.startswith("PARSE_FAILURE "))
    end = next(l for l in lines if l.startswith("EPISODE_END "))
    assert json.loads(fail.split(" ", 1)[1])["uid"] == "ge"
    e = json.loads(end.split(" ", 1)[1])
    assert e["reason"] == "parse" and e["success"] is False and e["turns"] == 1 and e["tokens"] > 0


def test_answer_parsing_cases_of_the_family():
    """The family's answer format, case by case: the call is the LAST fenced json block after the thinking; a block inside the
    thinking is no answer; an invalid block gives its reason and no call; without a thinking marker the whole text counts."""
    action = '{"x": 1.5}'
    text = f'<think>```json\n{{"x": 0}}\n```</think>first ```json\n{{"x": 0.5}}\n``` then ```json\n{action}\n```'
    assert extract_action(text) == {"x": 1.5}
    calls = get_parser("qwen3_8")(text)
    assert [(c.name, c.arguments) for c in calls] == [("env", {"x": 1.5})]
    with pytest.raises(ParseError, match="no fenced json block"):
        extract_action(f"<think>```json\n{action}\n```</think>no block here")
    assert get_parser("qwen3_8")(f"<think>```json\n{action}\n```</think>no block here") == []
    with pytest.raises(ParseError, match="invalid json"):
        extract_action('</think>```json\n{"x": }\n```')
    assert extract_action(f"plain ```json\n{action}\n```") == {"x": 1.5}


def test_cameras_of_different_sizes_take_their_own_block_lengths():
    """One observation, two cameras with pictures of different sizes: each block sits at its own run of placeholders."""
    from pear_b200.envs.tool import Observation
    from pear_b200.loop.episode import Episode
    from pear_b200.loop.vision_encoder import VisionEncoder
    from pear_b200.models.vision import FamilyVisionConfig, FamilyVisionTower

    tok = ByteTokenizer()
    enc = VisionEncoder(FamilyVisionTower(FamilyVisionConfig.tiny(out_hidden=8)).init_weights(0))
    loop = AgentLoop(None, None, tok, AgentLoopConfig(picture_positions="checkpoint"), {}, vision=enc)
    rng = np.random.default_rng(0)
    obs = Observation("state", [rng.integers(0, 256, (16, 24, 3), dtype=np.uint8), rng.integers(0, 256, (32, 8, 3), dtype=np.uint8)], ["front", "wrist"])
    ep = Episode(uid="u", session="0", family="f", env_args={})
    loop._append_user_turn(ep, obs, first=True)
    (p0, b0), (p1, b1) = ep.embeds
    assert b0.shape == (6, 8) and b1.shape == (4, 8) and ep.grids == [(2, 3), (4, 1)]
    assert all(t == tok.image_pad_id for t in ep.tokens[p0:p0 + 6]) and all(t == tok.image_pad_id for t in ep.tokens[p1:p1 + 4]) and p1 > p0 + 6
    pos = loop._positions(ep)
    assert pos.shape == (3, len(ep.tokens)) and pos[1, p1:p1 + 4].tolist() == [int(pos[0, p1]) + d for d in range(4)]  # a 4 x 1 block: rows advance
