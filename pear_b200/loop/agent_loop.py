"""The agent loop: one episode = one multi-turn conversation between the policy and an environment.

The state machine of upstream ``pear/agent_loop/agent_loop.py:24-242``:
PENDING -> GENERATING -> PROCESSING_TOOLS -> ... -> TERMINATED, with

* a token budget per EPISODE, not per turn: every generate call may use what is left (``:130``);
* end reasons ENV / PARSE / BUDGET (``episode.py:9-14``);
* up to ``max_restarts`` restarts of the whole trajectory when the environment process is lost (``:30, :50-66``);
* reward = the environment's success flag (``:70``);
* user turns merged into the running token list with response mask 0 and placeholder top-k heads, so the trainer sees
  one packed sequence per episode (``_resume_generating`` ``:198-229``);
* per-turn JSONL logs (``:178-196``).

The finished trajectory is written to the transfer queue under ``<uid>/<session>`` and sealed.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..envs.tool import EnvTool, Observation, episode_system_prompt, load_system_prompt
from ..rollout.engine import FinishReason, SamplingParams
from ..sim.env import EpisodeLost
from ..sim.server import ServerPool
from ..utils.files import append_jsonl
from ..utils.logging_utils import event, get_logger
from ..utils.tokenizer import ByteTokenizer
from .episode import EndReason, Episode, LoopState
from .protocol import ParseError, parse_answer, validate_action
from .tool_parser import get_parser


@dataclass
class AgentLoopConfig:
    token_budget: int = 512          # sampled tokens per episode
    max_turns: int = 16
    max_restarts: int = 2
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    topk_heads: int = 0              # rollout top-k head ids / log-probs kept for score centering
    max_model_len: int = 4096
    max_prompt_length: int = 0       # an episode whose first-turn prompt is longer ends at once (budget end, no sampled token); 0: no limit
    log_dir: Optional[str] = None
    # synthetic benchmarks with a random-init policy: play `synthetic_turns` turns with a no-op action whatever the answer
    # says, at most `turn_max_tokens` sampled tokens per turn (0: the episode budget), and draw the reward ("hash": a seeded
    # hash of the sampled tokens mapped to {0, 1}; "bernoulli:p": a seeded coin per trajectory) instead of the env's success
    # positions of picture rows: "sequential" (a row's position is its index) or "checkpoint" (the family's (temporal, row, column)
    # rule its pretrained checkpoints expect: needs pictures as pixels, whose grid is known; such requests take the engine's
    # per-request path)
    picture_positions: str = "sequential"
    tool_parser: str = "fenced_json"  # how an answer becomes the environment tool's call (`loop/tool_parser.py` registry)
    synthetic_turns: int = 0
    turn_max_tokens: int = 0
    synthetic_reward: Optional[str] = None


_log = get_logger("pear_b200.agent_loop")


class AgentLoop:
    def __init__(self, router, pool: ServerPool, tokenizer: ByteTokenizer, cfg: AgentLoopConfig, schemas: dict[str, dict],
                 queue=None, tracker=None, vision=None):
        """``vision``: a ``loop.vision_encoder.VisionEncoder`` for environments whose cameras deliver pixels."""
        self.router, self.pool, self.tok, self.cfg, self.vision = router, pool, tokenizer, cfg, vision
        self.schemas, self.queue, self.tracker = schemas, queue, tracker
        self.system_prompt = load_system_prompt()
        self.parse_calls = get_parser(cfg.tool_parser)

    # -- token bookkeeping --------------------------------------------------------------------------------------------
    def _append(self, ep: Episode, ids: list[int], mask: int, logprobs=None, topk_ids=None, topk_lps=None, version: int = 0) -> None:
        k = self.cfg.topk_heads
        ep.tokens += ids
        ep.response_mask += [mask] * len(ids)
        ep.logprobs += list(logprobs) if logprobs is not None else [0.0] * len(ids)
        ep.topk_ids += [list(r) for r in topk_ids] if topk_ids else [[0] * k for _ in ids]
        ep.topk_logprobs += [list(r) for r in topk_lps] if topk_lps else [[0.0] * k for _ in ids]
        ep.policy_versions += [version] * len(ids)

    def _append_user_turn(self, ep: Episode, obs: Observation, first: bool) -> None:
        ids: list[int] = []
        if first:
            ids += self.tok.render_turn("system", episode_system_prompt(self.system_prompt, obs))
        pixels = [f if (f.ndim == 3 and f.dtype == np.uint8) else None for f in obs.frames]
        if self.cfg.picture_positions == "checkpoint":
            if self.vision is None or any(p is None for p in pixels):
                raise ValueError("picture_positions=checkpoint needs cameras that deliver pixels and a vision encoder (the rows' grid must be known)")
            ep.grids += [self.vision.grid(p) for p in pixels]
        if self.vision is not None:
            obs.frames = self.vision.encode(obs.frames)
        elif any(f.ndim != 2 for f in obs.frames):
            raise ValueError("the environment delivers pixels: the agent loop needs a vision encoder (AgentLoopManager(vision=...))")
        counts = [int(f.shape[0]) for f in obs.frames]  # cameras of different sizes give blocks of different lengths
        turn = self.tok.render_turn("user", obs.text, images=len(obs.frames), image_tokens=counts, labels=obs.cameras or None)
        base = len(ep.tokens) + len(ids)
        # positions of the image pad runs inside the turn -> embedding blocks
        j, f = 0, 0
        while j < len(turn) and f < len(obs.frames):
            if turn[j] == self.tok.image_pad_id:
                ep.embeds.append((base + j, np.asarray(obs.frames[f], dtype=np.float32)))
                if pixels[f] is not None:  # a trainer with the tower in its graph recomputes this block from the picture
                    ep.images.append((base + j, pixels[f]))
                j += counts[f]
                f += 1
            else:
                j += 1
        self._append(ep, ids + turn + self.tok.generation_prompt(), 0)

    def _positions(self, ep: Episode):
        """[3, tokens] checkpoint positions of the episode so far (None under sequential positions or without pictures)."""
        if self.cfg.picture_positions != "checkpoint" or not ep.grids:
            return None
        from ..models.hybrid import mrope_positions

        return mrope_positions(torch.tensor(ep.tokens), ep.grids, self.tok.image_pad_id, merge=1)

    def _embeds(self, ep: Episode, hidden: int):
        if not ep.embeds:
            return None, None
        e = torch.zeros(len(ep.tokens), hidden)
        m = torch.zeros(len(ep.tokens), dtype=torch.bool)
        for pos, block in ep.embeds:
            e[pos:pos + block.shape[0]] = torch.from_numpy(block)
            m[pos:pos + block.shape[0]] = True
        return e, m

    def _log_turn(self, ep: Episode, state: LoopState, **extra) -> None:
        if self.cfg.log_dir:
            append_jsonl(f"{self.cfg.log_dir}/turns.jsonl", {"uid": ep.uid, "session": ep.session, "turn": ep.turns,
                                                            "state": state.value, "tokens": len(ep.tokens), **extra})

    # -- one episode --------------------------------------------------------------------------------------------------
    def run(self, uid: str, session: str, family: str, env_args: dict) -> Episode:
        for attempt in range(self.cfg.max_restarts + 1):
            ep = Episode(env_args=env_args, family=family, uid=uid, session=session, restarts=attempt)
            try:
                self._run_once(ep)
                break
            except EpisodeLost as e:
                self._log_turn(ep, LoopState.TERMINATED, lost=str(e), attempt=attempt)
                event(_log, "TRAJECTORY_RESTART", uid=ep.uid, session=ep.session, family=ep.family, attempt=attempt, reason=str(e)[:200])
                if attempt == self.cfg.max_restarts:
                    ep.end_reason, ep.success = EndReason.LOST, False
        self._publish(ep)
        event(_log, "EPISODE_END", uid=ep.uid, session=ep.session, family=ep.family, reason=ep.end_reason.value if ep.end_reason else None,
              success=bool(ep.success), turns=ep.turns, tokens=len(ep.tokens), response_tokens=ep.response_tokens, restarts=ep.restarts)
        return ep

    def _run_once(self, ep: Episode) -> None:
        cfg = self.cfg
        tool = EnvTool(self.pool, ep.family, log_path=f"{cfg.log_dir}/calls.jsonl" if cfg.log_dir else None)
        schema = self.schemas[ep.family]
        hidden = self.router.hidden_size
        state = LoopState.PENDING
        try:
            obs = tool.open(ep.env_args)
            self._append_user_turn(ep, obs, first=True)
            ep.prompt_len = len(ep.tokens)
            state = LoopState.GENERATING
            if cfg.max_prompt_length > 0 and ep.prompt_len > cfg.max_prompt_length:  # (upstream filters such rows out of the dataset)
                ep.end_reason, state = EndReason.BUDGET, LoopState.TERMINATED
            while state != LoopState.TERMINATED:
                if state == LoopState.GENERATING:
                    left = min(cfg.token_budget - ep.response_tokens, cfg.max_model_len - len(ep.tokens))
                    if cfg.turn_max_tokens > 0:
                        left = min(left, cfg.turn_max_tokens)
                    if cfg.synthetic_turns > 0 and ep.turns >= cfg.synthetic_turns:
                        ep.end_reason, state = EndReason.ENV, LoopState.TERMINATED
                        continue
                    if left <= 0 or ep.turns >= cfg.max_turns:
                        ep.end_reason, state = EndReason.BUDGET, LoopState.TERMINATED
                        continue
                    embeds, mask = self._embeds(ep, hidden)
                    params = SamplingParams(max_tokens=left, temperature=cfg.temperature, top_p=cfg.top_p, top_k=cfg.top_k,
                                            topk_logprobs=cfg.topk_heads, stop_token_ids=(self.tok.eos_id,) + tuple(getattr(self.tok, "extra_stop_ids", ())))
                    t0 = time.time()
                    positions = self._positions(ep)
                    extra = {} if positions is None else {"position_ids": positions}  # (routers without pictures never see the argument)
                    req = self.router.generate(list(ep.tokens), params, session=f"{ep.uid}/{ep.session}", embeds=embeds, embeds_mask=mask, **extra)
                    if req.finish == FinishReason.ABORTED:
                        ep.end_reason, state = EndReason.ABORTED, LoopState.TERMINATED
                        continue
                    self._append(ep, req.output, 1, req.logprobs, req.topk_ids or None, req.topk_logprobs or None, req.policy_version)
                    ep.turns += 1
                    self._log_turn(ep, state, sampled=len(req.output), seconds=round(time.time() - t0, 4), finish=req.finish.value)
                    if cfg.synthetic_turns > 0:  # the answer is not parsed: a no-op action keeps the episode going
                        action, state = {"move": 0}, LoopState.PROCESSING_TOOLS
                        continue
                    if req.finish == FinishReason.LENGTH:
                        ep.end_reason, state = EndReason.BUDGET, LoopState.TERMINATED
                        continue
                    answer = self.tok.decode([t for t in req.output if t != self.tok.eos_id])
                    try:
                        calls = self.parse_calls(answer)
                        if len(calls) != 1:  # one call to the environment per turn; none: the answer had no action
                            parse_answer(answer, schema)  # (raises with the reason when the default format finds none either)
                            raise ParseError(f"{len(calls)} tool calls in one answer")
                        action = calls[0].arguments
                        validate_action(action, schema)
                    except ParseError as e:
                        self._log_turn(ep, state, parse_error=str(e))
                        event(_log, "PARSE_FAILURE", uid=ep.uid, session=ep.session, turn=ep.turns, error=str(e)[:200])
                        ep.end_reason, state = EndReason.PARSE, LoopState.TERMINATED
                        continue
                    state = LoopState.PROCESSING_TOOLS
                else:  # PROCESSING_TOOLS
                    obs = tool.step(action)
                    if obs.done:
                        ep.success, ep.end_reason, state = obs.success, EndReason.ENV, LoopState.TERMINATED
                        continue
                    self._append(ep, self.tok.encode("\n"), 0)
                    self._append_user_turn(ep, obs, first=False)
                    state = LoopState.GENERATING
        finally:
            tool.close()

    def _reward(self, ep: Episode) -> float:
        mode = self.cfg.synthetic_reward
        if not mode:
            return float(ep.success)
        import hashlib

        if mode == "hash":
            sampled = np.asarray([t for t, m in zip(ep.tokens, ep.response_mask) if m], dtype=np.int64)
            return float(hashlib.blake2b(sampled.tobytes(), digest_size=8, key=b"pear-reward").digest()[0] & 1)
        if mode.startswith("bernoulli:"):
            p = float(mode.split(":", 1)[1])
            h = int.from_bytes(hashlib.blake2b(f"{ep.uid}/{ep.session}".encode(), digest_size=8, key=b"pear-reward").digest(), "little")
            return float((h >> 11) / float(1 << 53) < p)
        raise ValueError(f"unknown synthetic_reward {mode!r}")

    def _publish(self, ep: Episode) -> None:
        reward = self._reward(ep)
        if self.queue is not None:
            key = f"{ep.uid}/{ep.session}"
            self.queue.put_trajectory(key, {
                "tokens": np.asarray(ep.tokens, dtype=np.int64),
                "response_mask": np.asarray(ep.response_mask, dtype=np.int8),
                "rollout_logprobs": np.asarray(ep.logprobs, dtype=np.float32),
                # (explicit width: an episode lost before its first turn has no tokens, and -1 cannot be inferred from nothing)
                "topk_ids": np.asarray(ep.topk_ids, dtype=np.int64).reshape(len(ep.tokens), self.cfg.topk_heads),
                "topk_logprobs": np.asarray(ep.topk_logprobs, dtype=np.float32).reshape(len(ep.tokens), self.cfg.topk_heads),
                "embeds": [(p, b.astype(np.float16)) for p, b in ep.embeds],
                "images": list(ep.images),
                "position_ids": (lambda p: None if p is None else p.numpy().astype(np.int32))(self._positions(ep)),
                "policy_versions": np.asarray(ep.policy_versions, dtype=np.int32),
                "reward": reward, "prompt_len": ep.prompt_len,
            }, family=ep.family, end_reason=ep.end_reason.value if ep.end_reason else None, turns=ep.turns, restarts=ep.restarts)
        if self.tracker is not None:
            self.tracker.record(uid=ep.uid, session=ep.session, family=ep.family, reward=reward, turns=ep.turns,
                                end_reason=ep.end_reason.value if ep.end_reason else None, tokens=len(ep.tokens))
