"""Rollout engine: continuous batching over paged KV with prefix caching across rounds, host-DRAM offload of evicted
prefixes, chunked prefill, MTP speculative decoding and pause/abort/resume for weight sync.

It replaces the serving runtime the upstream builds on (vLLM V2 runner + scheduler + LMCache connector, wrapped by
``pear/rollout/server.py``) with the framework's own pieces:

* requests carry a ``session`` so a multi-turn episode hits the prefix its previous turn left behind (sticky routing,
  ``examples/.../run_stage1.sh:102-104``); every finished request publishes its full blocks, and the recurrent-state
  snapshot of its last full block, so the next turn resumes right after the previous answer;
* a step schedules decode/verify rows first, then prefill chunks up to ``max_num_batched_tokens`` (chunked prefill);
  when blocks run out the youngest running request is preempted (its blocks are released, it re-enters the queue and
  re-hits its own prefix);
* ``pause(abort=True)`` stops scheduling and returns every in-flight request as ABORTED with the tokens it has so far
  (the client resubmits, upstream patches 0044/0048); requests submitted while paused are rejected as aborted;
* ``update_weights`` loads new tensors in place, bumps the policy version, and invalidates the prefix cache and the
  host tier (``pear/rollout/lmcache.py:263-274``);
* per-request MTP acceptance counts and the counters the monitor scrapes are kept (patches 0051/0053,
  ``pear/monitor/metrics.py:88-97``).
"""

from __future__ import annotations

import itertools
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Optional

import torch

from ..utils import nvtx
from ..models.hybrid import HybridForCausalLM
from . import sampler as S
from .block_manager import NULL_BLOCK, BlockManager
from .host_tier import HostTier
from .model_runner import ModelRunner, SeqState, StepRow


class FinishReason(str, Enum):
    LENGTH = "length"
    STOP = "stop"
    ABORTED = "aborted"


@dataclass
class SamplingParams:
    max_tokens: int = 64
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    topk_logprobs: int = 0
    stop_token_ids: tuple = ()
    seed: Optional[int] = None


@dataclass
class Request:
    request_id: str
    prompt: list[int]
    params: SamplingParams
    session: Optional[str] = None
    embeds: Optional[torch.Tensor] = None  # [len(prompt), H] placeholder rows (vision embeddings)
    embeds_mask: Optional[torch.Tensor] = None
    # [3, len(prompt)] (temporal, row, column) positions of a prompt with pictures under the checkpoint's rule (None: every token's
    # position is its index); generated tokens continue one after the largest position of the prompt
    position_ids: Optional[torch.Tensor] = None
    arrival: float = field(default_factory=time.time)
    # -- runtime
    output: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    topk_ids: list[list[int]] = field(default_factory=list)
    topk_logprobs: list[list[float]] = field(default_factory=list)
    block_table: list[int] = field(default_factory=list)
    computed: int = 0  # tokens whose KV / state are in the caches
    cached_prefix: int = 0
    seq: Optional[SeqState] = None
    drafts: list[int] = field(default_factory=list)
    spec_drafted: int = 0
    spec_accepted: int = 0
    finish: Optional[FinishReason] = None
    policy_version: int = 0
    preemptions: int = 0

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output


@dataclass
class EngineConfig:
    num_blocks: int = 512
    block_size: int = 16
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 8192
    enable_prefix_caching: bool = True
    num_speculative_tokens: int = 0
    host_blocks: int = 0  # capacity of the host-DRAM tier in blocks (0: disabled)
    host_bytes: int = 0  # ... or in bytes (the tier holds as many blocks as fit); `host_blocks` wins when both are set
    host_numa_node: Optional[int] = None  # report the tier's locality to this node after it was touched
    state_interval_blocks: int = 0  # extra recurrent-state snapshots every N blocks during prefill (0: turn ends only)
    seed: int = 0
    fast_decode: bool = True  # on a GPU: decode / verify rows go through the batched GPU-resident step (rollout/fast_step.py)
    max_blocks_per_seq: int = 0  # width of the device block table of the fast step (0: num_blocks)


class RolloutEngine:
    def __init__(self, model: HybridForCausalLM, cfg: EngineConfig, device="cpu"):
        self.device = torch.device(device)
        self.model, self.cfg = model.eval().to(self.device), cfg
        n_slots = 2 * cfg.max_num_seqs + 64
        self.runner = ModelRunner(model, cfg.num_blocks, cfg.block_size, n_slots, device)
        self.host = None
        has_state = len(model.config.gdn_layers) > 0
        self.blocks = BlockManager(cfg.num_blocks, cfg.block_size, n_slots, cfg.enable_prefix_caching, needs_state=has_state)
        host_blocks = cfg.host_blocks
        if host_blocks <= 0 and cfg.host_bytes > 0:
            host_blocks = cfg.host_bytes // max(1, HostTier.bytes_per_block(self.runner.kv_tensors(), self.runner.state_tensors()))
        if host_blocks > 0:
            self.host = HostTier(host_blocks, self.runner.kv_tensors(), self.runner.state_tensors())
            self.host_locality = self.host.prefault(cfg.host_numa_node)
            self.blocks.host_tier = self.host
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: dict[str, Request] = {}
        self.paused = False
        self.policy_version = 0
        self.step_count = 0
        # sampling noise is drawn where the logits live: on a GPU the fused sampler / verifier run on the device
        self.gen = torch.Generator(device=self.device if self.device.type == "cuda" else "cpu").manual_seed(cfg.seed)
        self._ids = itertools.count()
        self.metrics = {"prompt_tokens": 0, "generation_tokens": 0, "preemptions": 0, "aborted": 0, "spec_drafted": 0,
                        "spec_accepted": 0, "steps": 0, "request_seconds": 0.0, "requests_finished": 0,
                        "first_token_seconds": 0.0, "first_tokens": 0}
        self.spec = cfg.num_speculative_tokens if model.mtp is not None else 0
        # the batched GPU-resident step for decode / verify rows (prefill chunks stay on the packed runner)
        self.fast = None
        self.symm = None  # set_symm_world(): tensor-parallel replicas hand their SymmWorld over before the first step
        self._fast_slot: dict[int, int] = {}  # id(request) -> batch slot of the fast step
        self._fast_free: list[int] = []
        self._fast_tables: dict[int, int] = {}  # id(request) -> block-table length already on the device
        self._fast_ok = (self.device.type == "cuda" and cfg.fast_decode and cfg.block_size == 16
                         and (not model.config.gdn_layers or (model.config.gdn_head_dim == 128 and model.config.conv_kernel == 4))
                         and model.config.head_dim in (64, 128, 256))

    # -- public API ---------------------------------------------------------------------------------------------------
    def add_request(self, prompt: list[int], params: Optional[SamplingParams] = None, session: Optional[str] = None,
                    request_id: Optional[str] = None, embeds=None, embeds_mask=None, position_ids=None) -> Request:
        req = Request(request_id or f"req-{next(self._ids)}", list(prompt), params or SamplingParams(), session, embeds, embeds_mask)
        if position_ids is not None:
            position_ids = torch.as_tensor(position_ids, dtype=torch.long)
            if tuple(position_ids.shape) != (3, len(prompt)):
                raise ValueError(f"position_ids must be [3, {len(prompt)}], got {tuple(position_ids.shape)}")
            req.position_ids = position_ids
        req.policy_version = self.policy_version
        if self.paused:  # the submission gate closes before the pause: the client resubmits later
            req.finish = FinishReason.ABORTED
            self.finished[req.request_id] = req
            self.metrics["aborted"] += 1
            return req
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def generate(self, prompts: list[list[int]], params: Optional[SamplingParams] = None, sessions=None) -> list[Request]:
        reqs = [self.add_request(p, params, sessions[i] if sessions else None) for i, p in enumerate(prompts)]
        while self.has_work():
            self.step()
        return reqs

    def pause(self, abort: bool = True) -> list[Request]:
        """Stop scheduling. ``abort``: in-flight requests end as ABORTED right away (not drained)."""
        self.paused = True
        out = []
        if abort:
            for req in list(self.running) + list(self.waiting):
                self._finish(req, FinishReason.ABORTED)
                out.append(req)
            self.waiting.clear()
            self.metrics["aborted"] += len(out)
        return out

    def resume(self) -> None:
        self.paused = False

    def update_weights(self, state: dict[str, torch.Tensor], version: Optional[int] = None) -> None:
        """In-place load (kernels reference the weights where they are), then invalidate every cached prefix."""
        assert not self.running, "pause(abort=True) before a weight update"
        own = dict(self.model.named_parameters())
        with torch.no_grad():
            for name, t in state.items():
                if name in own:
                    own[name].copy_(t.to(own[name].dtype))
        self.policy_version = version if version is not None else self.policy_version + 1
        if self.fast is not None:
            self.fast.repack()  # a no-op copy-wise when the parameters are views of the merged weights
        self.clear_kv_cache()

    def clear_kv_cache(self) -> int:
        return self.blocks.reset_prefix_cache(new_salt=f"v{self.policy_version}".encode())

    # -- sequence lifecycle -------------------------------------------------------------------------------------------
    def _admit(self, req: Request) -> bool:
        """Prefix lookup + state slot for a waiting request. False when resources are missing."""
        slot = self.blocks.allocate_slot()
        if slot is None:
            return False
        toks = req.tokens
        # the last token must be recomputed (its logits are needed), so look up at most len - 1 tokens
        hit = self.blocks.lookup(toks[: len(toks) - 1], extra_fn=self._extra_fn(req))
        req.block_table = list(hit.blocks)
        req.computed = req.cached_prefix = hit.tokens
        req.seq = SeqState(seq_id=id(req), slot=slot)
        if hit.state_slot is not None:
            self.runner.copy_state(hit.state_slot, slot)
        else:
            self.runner.zero_state(slot)
        if req.preemptions == 0:
            self.metrics["prompt_tokens"] += len(req.prompt)
        return True

    def _extra_fn(self, req: Request):
        if req.embeds is None:
            return None
        bs = self.cfg.block_size

        def extra(i: int) -> bytes:  # placeholder rows are content too: hash their bytes with the block
            m = req.embeds_mask[i * bs : (i + 1) * bs]
            if not bool(m.any()):
                return b""
            return req.embeds[i * bs : (i + 1) * bs][m].float().numpy().tobytes()

        return extra

    def _ensure_blocks(self, req: Request, upto_tokens: int) -> bool:
        need = (upto_tokens + self.cfg.block_size - 1) // self.cfg.block_size - len(req.block_table)
        if need <= 0:
            return True
        if not self.blocks.can_allocate(need):
            return False
        for _ in range(need):
            req.block_table.append(self.blocks.allocate())
        return True

    def _publish(self, req: Request, final: bool) -> None:
        """Publish the full blocks of the committed prefix; the last one (at a turn end, or every
        ``state_interval_blocks``) carries a snapshot of the recurrent state."""
        bs = self.cfg.block_size
        toks = req.tokens
        full = req.computed // bs
        if full == 0 or not self.cfg.enable_prefix_caching:
            return
        extra = self._extra_fn(req)
        parent = None
        for i in range(full):
            blk = req.block_table[i]
            b = self.blocks.blocks[blk]
            snap = None
            is_last = i == full - 1
            # the snapshot is valid only when the committed prefix ends exactly at this block's end
            at_boundary = is_last and req.computed == full * bs
            if at_boundary and self.blocks.needs_state and b.state_slot is None and (final or self._interval_hit(full)):
                snap = self.blocks.allocate_slot()
                if snap is not None:
                    self.runner.flush(req.seq)
                    self.runner.copy_state(req.seq.slot, snap)
            if b.hash is None or snap is not None:
                parent = self.blocks.publish(blk, parent, toks[i * bs : (i + 1) * bs], snap, extra(i) if extra else b"")
            else:
                parent = b.hash

    def _interval_hit(self, full_blocks: int) -> bool:
        n = self.cfg.state_interval_blocks
        return n > 0 and full_blocks % n == 0

    def _finish(self, req: Request, reason: FinishReason) -> None:
        req.finish = reason
        if reason != FinishReason.ABORTED:  # request latency from its arrival (queueing included), for the replica's metrics
            self.metrics["request_seconds"] += time.time() - req.arrival
            self.metrics["requests_finished"] += 1
        self._fast_release(req)
        if req.seq is not None:
            if reason != FinishReason.ABORTED:
                self.runner.flush(req.seq)
                # a turn end: commit the tail so the block boundary (if any) carries a snapshot
                self._publish(req, final=True)
            if self.host is not None and reason != FinishReason.ABORTED:
                hashes = [self.blocks.blocks[b].hash for b in req.block_table]
                slots = [self.blocks.blocks[b].state_slot for b in req.block_table]
                self.host.run_store(self.host.schedule_store(req.block_table, hashes, slots, session=req.session))
            for b in req.block_table:
                self.blocks.release(b)
            self.blocks.release_slot(req.seq.slot)
            req.block_table, req.seq = [], None
        if req in self.running:
            self.running.remove(req)
        self.finished[req.request_id] = req
        self.metrics["spec_drafted"] += req.spec_drafted
        self.metrics["spec_accepted"] += req.spec_accepted

    def _preempt(self, req: Request) -> None:
        self._fast_release(req)
        for b in req.block_table:
            self.blocks.release(b)
        self.blocks.release_slot(req.seq.slot)
        req.block_table, req.seq, req.computed, req.drafts = [], None, 0, []
        req.preemptions += 1
        self.running.remove(req)
        self.waiting.appendleft(req)
        self.metrics["preemptions"] += 1

    # -- one step -----------------------------------------------------------------------------------------------------
    def step(self) -> list[Request]:
        """Schedule and run one step; returns the requests that finished in it."""
        with nvtx.annotate("rollout/engine_step"):
            return self._step()

    def _step(self) -> list[Request]:
        if self.paused:
            return []
        cfg = self.cfg
        budget = cfg.max_num_batched_tokens
        rows: list[StepRow] = []
        plan: list[tuple[Request, int, bool]] = []  # (request, rows scheduled, is decode/verify)
        # 1. decode / verify rows of running requests whose prompt is fully computed
        fast_reqs = self._fast_candidates()
        for req in list(self.running):
            total = len(req.tokens)
            if req.computed < total - 1:
                continue
            if req.seq is None:  # preempted earlier in this loop
                continue
            if fast_reqs is not None:  # stepped by the batched GPU-resident step below
                continue
            n = 1 + len(req.drafts)
            planned = {id(p[0]) for p in plan}
            while not self._ensure_blocks(req, req.computed + n):
                # the youngest request that has no row in this step yet gives its blocks back (possibly `req` itself)
                victim = next((r for r in reversed(self.running) if id(r) not in planned and r.seq is not None), None)
                if victim is None:
                    break
                self._preempt(victim)
                if victim is req:
                    break
            if req.seq is None or not self._ensure_blocks(req, req.computed + n) or budget < n:
                continue
            toks = torch.tensor([req.tokens[-1]] + req.drafts, dtype=torch.long)
            rows.append(StepRow(req.seq, toks, req.computed, req.block_table, n, positions=self._row_positions(req, req.computed, n)))
            plan.append((req, n, True))
            budget -= n
        # 2. prefill chunks: running requests still in prefill, then newly admitted ones
        def add_prefill(req: Request) -> None:
            nonlocal budget
            total = len(req.tokens)
            remaining = (total - 1) - req.computed
            n = min(remaining, budget)
            if n <= 0:
                return
            last_chunk = n == remaining
            n_rows = n + (1 if last_chunk else 0)  # the final chunk also runs the last token to get its logits
            if last_chunk and budget < n_rows:
                n_rows, last_chunk = n, False
            if not self._ensure_blocks(req, req.computed + n_rows):
                return
            s = req.computed
            toks = torch.tensor(req.tokens[s : s + n_rows], dtype=torch.long)
            emb = msk = None
            if req.embeds is not None and s < len(req.prompt):
                e = min(s + n_rows, len(req.prompt))
                emb = torch.zeros(n_rows, req.embeds.shape[1])
                msk = torch.zeros(n_rows, dtype=torch.bool)
                emb[: e - s], msk[: e - s] = req.embeds[s:e], req.embeds_mask[s:e]
            rows.append(StepRow(req.seq, toks, s, req.block_table, 1 if last_chunk else 0, emb, msk, positions=self._row_positions(req, s, n_rows)))
            plan.append((req, n_rows, False))
            budget -= n_rows

        for req in self.running:
            if req.computed < len(req.tokens) - 1 and all(req is not p[0] for p in plan):
                add_prefill(req)
        while self.waiting and budget > 0 and len(self.running) < cfg.max_num_seqs:
            req = self.waiting[0]
            if not self._admit(req):
                break
            self.waiting.popleft()
            self.running.append(req)
            if len(req.tokens) == 1:  # nothing to prefill: decode right away next step
                continue
            add_prefill(req)
        if not rows:
            if fast_reqs:
                return self._fast_step(fast_reqs)
            if self.running and not any(True for _ in rows):
                # every running request is blocked on memory: preempt the youngest to make progress
                if len(self.running) > 1:
                    self._preempt(self.running[-1])
            return []
        speculative = any(is_dec and n > 1 for _, n, is_dec in plan)
        logits, resid, x_all, bounds = self.runner.forward(rows, speculative=speculative)
        self.step_count += 1
        self.metrics["steps"] += 1
        done: list[Request] = []
        lo = 0
        for i, (req, n, is_dec) in enumerate(plan):
            row = rows[i]
            if not is_dec:
                # prefill chunk: rows are committed; the final chunk's last row yields the first sampled token
                if self.spec > 0:
                    self._fill_drafter_kv(req, row, x_all[bounds[i] : bounds[i + 1]])
                if row.need_logits:
                    req.computed += n - 1
                    self._sample_rows(req, logits[lo : lo + 1], resid[lo : lo + 1], [], row)
                    lo += 1
                    if req.finish is None:
                        self._publish(req, final=False)
                else:
                    req.computed += n
                    if self._interval_hit(req.computed // cfg.block_size) and req.computed % cfg.block_size == 0:
                        self._publish(req, final=False)
            else:
                self._sample_rows(req, logits[lo : lo + n], resid[lo : lo + n], req.drafts, row)
                lo += n
            if req.finish is not None:
                done.append(req)
        if fast_reqs:
            done += self._fast_step([r for r in fast_reqs if r.finish is None and r.seq is not None])
        return done

    # -- the batched GPU-resident step --------------------------------------------------------------------------------------
    def set_symm_world(self, symm) -> None:
        """Tensor-parallel replica: the fast step reduces its row-parallel partials through this ``SymmWorld``."""
        self.symm = symm

    def _fast_candidates(self):
        """Decode-phase requests when ALL of them can take the fast step (one temperature > 0, plain sampling, at most 32 top
        log-probs per token); None when the step has to stay on the packed runner."""
        from ..models import hybrid

        if not self._fast_ok or (hybrid.tensor_parallel_active() and self.symm is None):
            return None
        reqs = [r for r in self.running if r.seq is not None and r.output and r.computed >= len(r.tokens) - 1]
        if not reqs:
            return []
        p0 = reqs[0].params
        if p0.temperature <= 0.0 or any(r.params.temperature != p0.temperature or r.params.top_p < 1.0 or r.params.top_k > 0 or r.params.topk_logprobs > 32 or r.params.seed is not None or r.position_ids is not None
                                        for r in reqs):
            for r in list(self.running):
                self._fast_release(r)
            return None
        return reqs

    def _fast_init(self, temperature: float, topk: bool = False) -> None:
        from .fast_step import FastDecoder

        cfg, rn = self.cfg, self.runner
        width = cfg.max_blocks_per_seq or cfg.num_blocks
        self.fast = FastDecoder(self.model, rn.k_cache, rn.v_cache, rn.rec_state, rn.mtp_k if rn.has_mtp else [], rn.mtp_v if rn.has_mtp else [],
                                num_slots=2 * cfg.max_num_seqs + 64, max_batch=cfg.max_num_seqs, n_draft=self.spec, max_blocks_per_seq=width,
                                temperature=temperature, seed=cfg.seed, symm=self.symm, topk_logprobs=topk)
        self._fast_free = list(range(cfg.max_num_seqs - 1, -1, -1))

    def _fast_release(self, req: Request, commit: Optional[int] = None) -> None:
        """Take a request out of the fast batch: its committed rows (``commit`` of the last block when the sequence was
        cut short of what the device accepted) are replayed into the recurrent state and the conv window goes back to
        the runner's state slot (a snapshot or the packed runner continues from there)."""
        b = self._fast_slot.pop(id(req), None)
        if b is None:
            return
        self._fast_tables.pop(id(req), None)
        conv = self.fast.release(b, commit)
        if req.seq is not None:
            for li, rows in conv.items():
                self.runner.conv_state[li][req.seq.slot].copy_(rows)
        self._fast_free.append(b)

    def _shared_prefix_groups(self, reqs: list[Request]) -> list:
        """Sequences whose block tables start with the same pages (samples of one prompt, turns of one session that hit
        the prefix cache): (batch slots, shared tokens) per group, for the attention kernel that reads shared pages once."""
        buckets: dict[int, list[Request]] = {}
        for r in reqs:
            if r.block_table:
                buckets.setdefault(r.block_table[0], []).append(r)
        groups = []
        bs = self.cfg.block_size
        for members in buckets.values():
            if len(members) < 2:
                continue
            first = members[0].block_table
            common = min(len(m.block_table) for m in members)
            for m in members[1:]:
                n = 0
                while n < common and m.block_table[n] == first[n]:
                    n += 1
                common = n
            tokens = min(common * bs, min(m.computed for m in members))
            if tokens >= 256:
                groups.append(([self._fast_slot[id(m)] for m in members], tokens))
        return groups

    def _fast_step(self, reqs: list[Request]) -> list[Request]:
        if not reqs:
            return []
        temp = reqs[0].params.temperature
        want_topk = any(r.params.topk_logprobs > 0 for r in reqs)
        if self.fast is not None and want_topk and not self.fast.topk:
            # the decoder was built without the top log-prob kernels (they are part of its captured graph): rebuild it with them
            for r in list(self.running):
                self._fast_release(r)
            self.fast = None
        if self.fast is None:
            self._fast_init(temp, topk=want_topk)
        elif self.fast.temperature != temp:
            self.fast.set_temperature(temp)
        fast, T = self.fast, 1 + self.spec
        active: list[Request] = []
        for req in reqs:
            if not self._ensure_blocks(req, req.computed + 2 * T):
                if id(req) not in self._fast_slot:
                    continue  # joins when pages are free again
                if not self._ensure_blocks(req, req.computed + T):
                    self._fast_release(req)
                    self._preempt(req)
                    continue
            if id(req) not in self._fast_slot:
                if not self._fast_free:
                    continue
                b = self._fast_free.pop()
                self.runner.flush(req.seq)
                conv = {li: self.runner.conv_state[li][req.seq.slot] for li in self.runner.gdn_layers}
                fast.assign(b, req.seq.slot, req.computed, req.block_table, req.tokens[-1], conv, drafts=req.drafts)
                req.drafts = []
                self._fast_slot[id(req)] = b
                self._fast_tables[id(req)] = len(req.block_table)
            elif self._fast_tables[id(req)] != len(req.block_table):
                fast.graph_sync()
                fast.set_block_table(self._fast_slot[id(req)], req.block_table)
                self._fast_tables[id(req)] = len(req.block_table)
            active.append(req)
        if not active:
            return []
        members = tuple(sorted((self._fast_slot[id(r)], r.block_table[0] if r.block_table else -1) for r in active))
        if members != getattr(self, "_fast_members", None):  # batch membership changed: regroup the sequences that share pages
            self._fast_members = members
            fast.set_shared_prefixes(self._shared_prefix_groups(active))
        fast.step()
        res = fast.results()
        fast.check()
        self.step_count += 1
        self.metrics["steps"] += 1
        done: list[Request] = []
        for req in active:
            b = self._fast_slot[id(req)]
            if int(res.nonfinite[b]) > 0:
                raise S.NonFiniteLogits(self.step_count, [b], [req.request_id])
            acc = int(res.accepted[b])
            req.computed += acc + 1
            req.spec_drafted += self.spec
            req.spec_accepted += acc
            p = req.params
            for j in range(acc + 1):
                t = int(res.tokens[b, j])
                req.output.append(t)
                req.logprobs.append(float(res.logprobs[b, j]))
                if p.topk_logprobs > 0:
                    req.topk_ids.append(res.topk_ids[b, j, : p.topk_logprobs].tolist())
                    req.topk_logprobs.append(res.topk_logprobs[b, j, : p.topk_logprobs].tolist())
                self.metrics["generation_tokens"] += 1
                reason = FinishReason.STOP if t in p.stop_token_ids else (FinishReason.LENGTH if len(req.output) >= p.max_tokens else None)
                if reason is not None:
                    # tokens the device committed past this one are not part of the sequence: the caches are cut back to here
                    req.computed -= acc - j
                    self._fast_release(req, commit=j + 1)
                    self._finish(req, reason)
                    done.append(req)
                    break
        return done

    # -- sampling / verification / drafting -----------------------------------------------------------------------------
    @staticmethod
    def _row_positions(req: Request, start: int, n: int) -> Optional[torch.Tensor]:
        """[3, n] positions of tokens ``start .. start + n`` of a request that carries its own prompt positions (else None: the
        runner counts from ``start``): prompt tokens from the table, later tokens one after another past the prompt's largest."""
        if req.position_ids is None:
            return None
        p = req.position_ids
        n_prompt = p.shape[1]
        after = int(p.max()) + 1 if n_prompt else 0
        idx = torch.arange(start, start + n)
        late = (after + (idx - n_prompt)).clamp(min=0).expand(3, -1)
        return torch.where((idx < n_prompt)[None], p[:, idx.clamp(max=max(n_prompt - 1, 0))], late)

    def _generator(self, req: Request) -> torch.Generator:
        """The engine's generator, or the request's own when it carries a seed: such a request draws the same tokens whatever
        else is in the batch (it stays on the per-request sampling path; the batched step draws from one counter stream)."""
        if req.params.seed is None:
            return self.gen
        g = getattr(req, "_gen", None)
        if g is None:
            g = torch.Generator(device=self.gen.device).manual_seed(int(req.params.seed))
            req._gen = g
        return g

    def _sample_rows(self, req: Request, logits: torch.Tensor, resid: torch.Tensor, drafts: list[int], row: StepRow) -> None:
        p = req.params
        bad = S.count_nonfinite(logits)
        if bool((bad > 0).any()):
            raise S.NonFiniteLogits(self.step_count, torch.nonzero(bad).flatten().tolist(), [req.request_id])
        if drafts:
            out = S.verify_greedy_drafts(logits[None], torch.tensor([drafts], device=logits.device), p.temperature, p.topk_logprobs, self._generator(req))
            acc = int(out.accepted[0])
            new = [int(t) for t in out.tokens[0, : acc + 1]]
            lps = [float(v) for v in out.logprobs[0, : acc + 1]]
            tk_i = [out.topk_ids[0, j].tolist() for j in range(acc + 1)] if out.topk_ids is not None else []
            tk_l = [out.topk_logprobs[0, j].tolist() for j in range(acc + 1)] if out.topk_logprobs is not None else []
            req.spec_drafted += len(drafts)
            req.spec_accepted += acc
        else:
            so = S.sample(logits[-1:], p.temperature, p.top_p, p.top_k, p.topk_logprobs, self._generator(req))
            acc, new, lps = 0, [int(so.tokens[0])], [float(so.logprobs[0])]
            tk_i = [so.topk_ids[0].tolist()] if so.topk_ids is not None else []
            tk_l = [so.topk_logprobs[0].tolist()] if so.topk_logprobs is not None else []
        committed = acc + 1  # rows [x0, accepted drafts] enter the state
        if row.need_logits > 1 or drafts:
            self.runner.commit(req.seq, committed)
        req.computed += committed if (drafts or row.tokens.shape[0] == 1) else 1
        req.seq.mtp_hidden = resid[acc]
        if not req.output:  # time to the first token, from the request's arrival
            self.metrics["first_token_seconds"] += time.time() - req.arrival
            self.metrics["first_tokens"] += 1
        for j, t in enumerate(new):
            req.output.append(t)
            req.logprobs.append(lps[j])
            if tk_i:
                req.topk_ids.append(tk_i[j])
                req.topk_logprobs.append(tk_l[j])
            self.metrics["generation_tokens"] += 1
            if t in p.stop_token_ids:
                self._finish(req, FinishReason.STOP)
                return
            if len(req.output) >= p.max_tokens:
                self._finish(req, FinishReason.LENGTH)
                return
        req.drafts = self._draft(req, row, resid, acc, new) if self.spec > 0 else []

    def _fill_drafter_kv(self, req: Request, row: StepRow, x_rows: torch.Tensor) -> None:
        """The drafter's KV of a prefill chunk: position p of the prompt pairs the main model's residual at p with the
        embedding of prompt token p + 1, so every chunk row whose next token is part of the prompt goes through one MTP pass
        (the row of the last prompt token is done by ``_draft`` once its successor has been sampled). Without this the
        drafter would attend over an empty cache for the whole prompt and propose from the generated tokens alone."""
        toks = req.tokens
        m = min(x_rows.shape[0], len(toks) - 1 - row.start)
        if m <= 0:
            return
        nxt = torch.tensor(toks[row.start + 1 : row.start + 1 + m], dtype=torch.long)
        self.runner.mtp_forward(StepRow(req.seq, nxt, row.start, req.block_table, 0, positions=self._row_positions(req, row.start, m)), nxt, x_rows[:m])

    def _draft(self, req: Request, row: StepRow, resid: torch.Tensor, acc: int, new: list[int]) -> list[int]:
        """MTP drafts for the next step: first a pass over the rows committed in this step (it fills the drafter's KV
        pages and predicts the token after ``new[-1]``), then greedy chained passes on the drafter's own output."""
        toks = req.tokens
        n_commit = acc + 1
        first = req.computed - n_commit  # position of the first committed row
        nxt = torch.tensor(toks[first + 1 : first + 1 + n_commit], dtype=torch.long)
        sub = StepRow(req.seq, nxt, first, req.block_table, 0, positions=self._row_positions(req, first, n_commit))
        if not self._ensure_blocks(req, req.computed + self.spec + 1):
            return []
        logits, r = self.runner.mtp_forward(sub, nxt, resid[:n_commit] if resid.shape[0] >= n_commit else resid[-1:].expand(n_commit, -1))
        drafts = [int(logits[-1].argmax())]
        hidden = r[-1:]
        for j in range(1, self.spec):
            pos = req.computed + j - 1
            sub = StepRow(req.seq, torch.tensor(drafts[-1:]), pos, req.block_table, 0, positions=self._row_positions(req, pos, 1))
            logits, hidden = self.runner.mtp_forward(sub, torch.tensor(drafts[-1:]), hidden)
            drafts.append(int(logits[-1].argmax()))
        return drafts

    def stats(self) -> dict:
        out = dict(self.metrics)
        out.update(self.blocks.stats())
        if self.host is not None:
            out.update(self.host.stats())
        out.update(num_running=len(self.running), num_waiting=len(self.waiting), policy_version=self.policy_version)
        return out
