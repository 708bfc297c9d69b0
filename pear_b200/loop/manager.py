"""Agent-loop manager (upstream ``pear/agent_loop/manager.py:14-41``): starts the environment server pools, owns a
least-in-flight router over the rollout replicas, and runs prompt groups on a pool of worker threads, dealing the
sessions of successive dispatches round-robin over the workers (so one slow group never pins a worker's whole queue)."""

from __future__ import annotations

import itertools
import queue
import threading
from concurrent.futures import Future
from typing import Optional

from ..sim.server import ServerPool
from ..utils.tokenizer import ByteTokenizer
from .agent_loop import AgentLoop, AgentLoopConfig


class Router:
    """Least-in-flight routing over rollout replicas; a session sticks to the replica that holds its prefix."""

    def __init__(self, servers: list, hidden_size: int):
        self.servers, self.hidden_size = servers, hidden_size
        self.inflight = [0] * len(servers)
        self.sticky: dict[str, int] = {}
        self.lock = threading.Lock()

    def _pick(self, session: Optional[str]) -> int:
        with self.lock:
            if session is not None and session in self.sticky:
                i = self.sticky[session]
            else:
                i = min(range(len(self.servers)), key=lambda j: self.inflight[j])
                if session is not None:
                    self.sticky[session] = i
            self.inflight[i] += 1
            return i

    def generate(self, prompt, params, session=None, embeds=None, embeds_mask=None, position_ids=None):
        i = self._pick(session)
        try:
            if position_ids is None:
                return self.servers[i].generate(prompt, params, session=session, embeds=embeds, embeds_mask=embeds_mask)
            return self.servers[i].generate(prompt, params, session=session, embeds=embeds, embeds_mask=embeds_mask, position_ids=position_ids)
        finally:
            with self.lock:
                self.inflight[i] -= 1

    def forget(self, session: str) -> None:
        with self.lock:
            self.sticky.pop(session, None)


class AgentLoopManager:
    def __init__(self, servers: list, hidden_size: int, env_families: dict[str, dict], cfg: AgentLoopConfig, queue_=None,
                 tracker=None, num_workers: int = 4, tokenizer: Optional[ByteTokenizer] = None, vision=None):
        """``env_families``: family -> {"env_path": dotted class path, "mode": "stateless"|"stateful", ...Server kwargs}; with
        ``"urls": [...]`` the family is served by environment hosts in other processes (``sim/server.py: main``) and only its
        action schema is taken from the class here."""
        self.pool = ServerPool()
        schemas = {}
        for family, spec in env_families.items():
            spec = dict(spec)
            env_path = spec.pop("env_path")
            mode = spec.pop("mode", "stateless")
            urls = spec.pop("urls", None)
            if urls:
                self.pool.connect(family, list(urls))
            else:
                self.pool.start(family, env_path, mode, **spec)
            module, _, name = env_path.rpartition(".")
            schemas[family] = getattr(__import__(module, fromlist=[name]), name).action_schema()
        self.router = Router(servers, hidden_size)
        self.loop = AgentLoop(self.router, self.pool, tokenizer or ByteTokenizer(), cfg, schemas, queue_, tracker, vision=vision)
        self.jobs: "queue.Queue" = queue.Queue()
        self.cancelled: set[str] = set()
        self.errors: list[str] = []
        self.stop_flag = False
        self._rr = itertools.count()
        self.worker_queues = [queue.Queue() for _ in range(num_workers)]
        self.workers = [threading.Thread(target=self._work, args=(q,), daemon=True, name=f"agent-loop-{i}")
                        for i, q in enumerate(self.worker_queues)]
        for w in self.workers:
            w.start()

    def _work(self, q: "queue.Queue") -> None:
        while not self.stop_flag:
            try:
                job = q.get(timeout=0.1)
            except queue.Empty:
                continue
            uid, session, family, env_args, fut = job
            if uid in self.cancelled:
                fut.cancel()
                continue
            try:
                fut.set_result(self.loop.run(uid, session, family, env_args))
            except BaseException as e:  # noqa: BLE001 - recorded so that the trainer fails fast instead of waiting for a group forever
                import traceback
                self.errors.append(f"{uid}/{session}: {type(e).__name__}: {e}\n{traceback.format_exc()}")
                fut.set_exception(e)
            finally:
                self.router.forget(f"{uid}/{session}")

    def dispatch_group(self, uid: str, family: str, env_args: dict, sessions: list[str]) -> list[Future]:
        """Run the sessions of one prompt group; sessions are dealt round-robin over the workers."""
        futs = []
        for s in sessions:
            fut: Future = Future()
            self.worker_queues[next(self._rr) % len(self.worker_queues)].put((uid, s, family, env_args, fut))
            futs.append(fut)
        return futs

    def cancel_group(self, uid: str) -> None:
        self.cancelled.add(uid)

    def close(self) -> None:
        self.stop_flag = True
        for w in self.workers:
            w.join(timeout=5)
        self.pool.close()
