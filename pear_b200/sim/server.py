"""Simulator servers: supervised environment subprocesses lent to episodes by a pool.

The role of upstream ``pear/sim/server.py`` (Ray-actor ``ServerPool`` on the head lending ``Server`` actors that
supervise simulator subprocesses over pipes), ``process.py`` and ``client.py``, without Ray: a ``Server`` owns one
subprocess per slot and talks to it over a pipe; a watchdog restarts ended processes; a call that exceeds its timeout
kills the process and raises ``EpisodeLost`` (``server.py:169-182``, ``process.py:122-134``); a stateless call is
retried once on another process (``:80-94``); a process that fails its first start three times fails the run
(``:37, :146-154``). ``ServerPool.acquire / release`` hands processes to episodes (``:262, :266``).

All failure paths are host-side: nothing here touches a GPU.
"""

from __future__ import annotations

import importlib
import json
import multiprocessing as mp
import threading
import time
import traceback
from dataclasses import dataclass
from typing import Any, Optional

from ..utils.process import die_with_parent
from .env import EpisodeLost, StatefulEnv, StatelessEnv

MAX_FIRST_START_FAILURES = 3


def _load(path: str):
    module, _, name = path.rpartition(".")
    return getattr(importlib.import_module(module), name)


def _worker(conn, env_path: str, mode: str, kwargs: dict) -> None:
    """Child process: serve calls from the pipe until it closes."""
    die_with_parent()
    try:
        env_cls = _load(env_path)
        host = StatelessEnv(env_cls, **kwargs) if mode == "stateless" else StatefulEnv(env_cls, **kwargs)
        conn.send(("ready", None))
    except Exception:  # noqa: BLE001
        conn.send(("error", traceback.format_exc()))
        return
    while True:
        try:
            msg = conn.recv()
        except (EOFError, OSError):
            return
        if msg is None:
            return
        method, args = msg
        try:
            conn.send(("ok", getattr(host, method)(*args)))
        except EpisodeLost as e:
            conn.send(("lost", str(e)))
        except Exception:  # noqa: BLE001
            conn.send(("error", traceback.format_exc()))


@dataclass
class _Slot:
    index: int
    proc: Optional[mp.Process] = None
    conn: Any = None
    busy: bool = False
    starts: int = 0
    ever_ready: bool = False
    episode: Optional[str] = None


class StartFailure(RuntimeError):
    pass


class Server:
    """Supervises ``num_processes`` environment subprocesses of one family."""

    def __init__(self, env_path: str, mode: str = "stateless", num_processes: int = 2, call_timeout_s: float = 30.0,
                 start_timeout_s: float = 60.0, env_kwargs: Optional[dict] = None, name: str = "server"):
        self.env_path, self.mode, self.name = env_path, mode, name
        self.call_timeout_s, self.start_timeout_s = call_timeout_s, start_timeout_s
        self.env_kwargs = env_kwargs or {}
        self.ctx = mp.get_context("spawn")
        self.lock = threading.Condition()
        self.slots = [_Slot(i) for i in range(num_processes)]
        self.failed: Optional[str] = None
        self.restarts = 0
        self.closed = False
        for s in self.slots:
            self._start(s)
        self.watchdog = threading.Thread(target=self._watch, daemon=True, name=f"{name}-watchdog")
        self.watchdog.start()

    # -- process lifecycle --------------------------------------------------------------------------------------------
    def _start(self, s: _Slot) -> None:
        parent, child = self.ctx.Pipe()
        s.proc = self.ctx.Process(target=_worker, args=(child, self.env_path, self.mode, self.env_kwargs), daemon=True)
        s.proc.start()
        child.close()
        s.conn, s.starts = parent, s.starts + 1
        ok = parent.poll(self.start_timeout_s)
        status = parent.recv() if ok else ("error", "start timed out")
        if status[0] != "ready":
            self._kill(s)
            if not s.ever_ready and s.starts >= MAX_FIRST_START_FAILURES:
                self.failed = f"{self.name}: process {s.index} failed its first start {s.starts} times: {status[1]}"
                raise StartFailure(self.failed)
            return self._start(s)
        s.ever_ready = True

    def _kill(self, s: _Slot) -> None:
        try:
            if s.conn is not None:
                s.conn.close()
        except OSError:
            pass
        if s.proc is not None and s.proc.is_alive():
            s.proc.kill()
            s.proc.join(5)
        s.proc, s.conn, s.episode = None, None, None

    def _watch(self) -> None:
        while not self.closed:
            time.sleep(0.2)
            with self.lock:
                for s in self.slots:
                    if not s.busy and (s.proc is None or not s.proc.is_alive()) and not self.closed and self.failed is None:
                        try:
                            self._kill(s)
                            self._start(s)
                            self.restarts += 1
                        except StartFailure:
                            pass
                self.lock.notify_all()

    # -- calls --------------------------------------------------------------------------------------------------------
    def _call(self, s: _Slot, method: str, args: tuple, timeout_s: Optional[float] = None):
        try:
            s.conn.send((method, args))
            if not s.conn.poll(timeout_s or self.call_timeout_s):
                raise TimeoutError(f"{self.name}: {method} exceeded {timeout_s or self.call_timeout_s}s")
            status, payload = s.conn.recv()
        except (TimeoutError, EOFError, OSError, BrokenPipeError) as e:
            with self.lock:
                self._kill(s)  # the watchdog starts a fresh process
            raise EpisodeLost(str(e)) from e
        if status == "ok":
            return payload
        if status == "lost":
            raise EpisodeLost(payload)
        raise RuntimeError(f"{self.name}: environment raised\n{payload}")

    def acquire(self, episode: Optional[str] = None, timeout_s: float = 60.0) -> _Slot:
        deadline = time.time() + timeout_s
        with self.lock:
            while True:
                if self.failed:
                    raise StartFailure(self.failed)
                for s in self.slots:
                    if not s.busy and s.proc is not None and s.proc.is_alive():
                        s.busy, s.episode = True, episode
                        return s
                if not self.lock.wait(max(0.0, min(0.5, deadline - time.time()))) and time.time() > deadline:
                    raise TimeoutError(f"{self.name}: no free environment process")

    def release(self, s: _Slot) -> None:
        with self.lock:
            s.busy, s.episode = False, None
            self.lock.notify_all()

    def rollout(self, args: dict, actions: list[dict]) -> dict:
        """Stateless call, retried once on another process when the first one is lost."""
        last: Optional[Exception] = None
        for _ in range(2):
            s = self.acquire()
            try:
                return self._call(s, "rollout", (args, actions))
            except EpisodeLost as e:
                last = e
            finally:
                self.release(s)
        raise EpisodeLost(f"{self.name}: stateless call lost twice: {last}")

    def close(self) -> None:
        self.closed = True
        with self.lock:
            for s in self.slots:
                try:
                    if s.conn is not None:
                        s.conn.send(None)
                except OSError:
                    pass
                self._kill(s)


class ServerPool:
    """Servers per environment family; episodes borrow a process through it."""

    def __init__(self) -> None:
        self.servers: dict[str, Server] = {}

    def start(self, family: str, env_path: str, mode: str = "stateless", **kwargs) -> Server:
        if family not in self.servers:
            self.servers[family] = Server(env_path, mode, name=family, **kwargs)
        return self.servers[family]

    def connect(self, family: str, urls: list[str], **kwargs) -> "RemoteServer":
        """The family is served by environment hosts in other processes (``python -m pear_b200.sim.server``)."""
        if family not in self.servers:
            self.servers[family] = RemoteServer(family, urls, **kwargs)
        return self.servers[family]

    def get(self, family: str) -> Server:
        return self.servers[family]

    def capacity(self, family: str) -> int:
        srv = self.servers[family]
        return srv.capacity() if isinstance(srv, RemoteServer) else len(srv.slots)

    def close(self) -> None:
        for s in self.servers.values():
            s.close()
        self.servers.clear()


def encode_arrays(obj):
    """JSON form of a rollout result: numpy arrays (camera frames, embedding blocks) become base64 with dtype and shape."""
    import base64

    import numpy as np

    if isinstance(obj, np.ndarray):
        return {"__ndarray__": base64.b64encode(np.ascontiguousarray(obj).tobytes()).decode(), "dtype": str(obj.dtype), "shape": list(obj.shape)}
    if isinstance(obj, dict):
        return {k: encode_arrays(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [encode_arrays(v) for v in obj]
    if isinstance(obj, np.generic):
        return obj.item()
    return obj


def decode_arrays(obj):
    import base64

    import numpy as np

    if isinstance(obj, dict):
        if "__ndarray__" in obj:
            return np.frombuffer(base64.b64decode(obj["__ndarray__"]), dtype=np.dtype(obj["dtype"])).reshape(obj["shape"]).copy()
        return {k: decode_arrays(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [decode_arrays(v) for v in obj]
    return obj


class RemoteServer:
    """A family's environment hosts behind the interface episodes use on a local :class:`Server` (stateless families: every call
    replays the action history, so any host can answer any call). A host that does not answer is skipped for a while and the
    call goes to the next one; when none answers the episode is lost (the agent loop restarts it). Upstream's clients route
    around dead server actors the same way (pear/sim/client.py:76-86)."""

    mode = "stateless"

    def __init__(self, family: str, urls: list[str], call_timeout_s: float = 60.0, retry_after_s: float = 10.0):
        import itertools
        import threading

        import requests

        self.name, self.urls, self.timeout, self.retry_after = family, [u.rstrip("/") for u in urls], call_timeout_s, retry_after_s
        self._requests, self._local = requests, threading.local()
        self._next = itertools.count()
        self.down: dict[str, float] = {}
        self.slots: list = []
        self.failovers = 0

    def _session(self):
        s = getattr(self._local, "s", None)
        if s is None:
            s = self._local.s = self._requests.Session()
        return s

    def capacity(self) -> int:
        total = 0
        for u in self.urls:
            try:
                total += int(self._session().get(u + "/capacity", timeout=5).json().get(self.name, 0))
            except Exception:  # noqa: BLE001 - a host that is down lends nothing
                pass
        return total

    def rollout(self, args: dict, actions: list[dict]) -> dict:
        import time

        start = next(self._next)
        order = [self.urls[(start + i) % len(self.urls)] for i in range(len(self.urls))]
        now = time.time()
        live = [u for u in order if self.down.get(u, 0.0) <= now] or order  # all marked down: try them anyway
        last = None
        for i, u in enumerate(live):
            try:
                r = self._session().post(u + "/rollout", json={"family": self.name, "args": args, "actions": actions}, timeout=self.timeout)
                body = r.json()
                if r.status_code == 200 and "lost" not in body:
                    self.down.pop(u, None)
                    return decode_arrays(body)
                last = body.get("lost") or f"HTTP {r.status_code}"
            except Exception as e:  # noqa: BLE001 - connection refused / reset / timed out: the host is gone or stuck
                last = repr(e)
                self.down[u] = time.time() + self.retry_after
            if i + 1 < len(live):
                self.failovers += 1
        raise EpisodeLost(f"{self.name}: no environment host answered ({last})")

    def close(self) -> None:
        pass


def http_app(pool: ServerPool):
    """The environment host's API: POST /rollout {family, args, actions} replays an action history in a borrowed process
    (the stateless contract of ``sim/env.py``), GET /capacity, GET /health."""
    from fastapi import FastAPI

    app = FastAPI(title="pear_b200 environment host")

    @app.get("/health")
    def health() -> dict:
        return {"ok": True, "families": sorted(pool.servers)}

    @app.get("/capacity")
    def capacity() -> dict:
        return {f: pool.capacity(f) for f in pool.servers}

    @app.post("/rollout")
    def rollout(body: dict) -> dict:
        try:
            return encode_arrays(pool.get(body["family"]).rollout(body.get("args", {}), body.get("actions", [])))
        except EpisodeLost as e:  # the host's own processes were lost twice: the client tries another host
            return {"lost": str(e)}

    return app


def main(argv=None) -> int:
    """``python -m pear_b200.sim.server --family synthetic=pear_b200.envs.synthetic.SyntheticEnv --port 8200``: an environment
    host as a process of its own (the env role of ``launch/roles.py``): supervised simulator subprocesses behind a small HTTP
    API. ``--check`` starts the pool, runs one empty rollout per family and exits."""
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--family", action="append", default=[], help="name=import.path.EnvClass (repeatable)")
    ap.add_argument("--processes", type=int, default=2)
    ap.add_argument("--env-kwargs", default="{}", help="JSON of the environment class's constructor arguments")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8200)
    ap.add_argument("--check", action="store_true")
    args, rest = ap.parse_known_args(argv)
    families = dict(f.split("=", 1) for f in args.family) or {"synthetic": "pear_b200.envs.synthetic.SyntheticEnv"}
    if args.env_kwargs == "{}" and not args.family:
        # the launcher passes the recipe's overrides to every role: the default synthetic family draws its placeholder rows at the
        # policy model's width, as the training entry's own environment processes do
        kv = dict(o.split("=", 1) for o in rest if "=" in o and not o.startswith("-"))
        path = kv.get("actor_rollout_ref.model.path")
        if path:
            from ..models import io as model_io
            from ..models.config import HybridConfig

            mcfg = getattr(HybridConfig, path.split(":", 1)[1])() if path.startswith("preset:") else model_io.load_config(path)
            args.env_kwargs = json.dumps({"hidden": mcfg.hidden_size, "tokens_per_image": 4})
    pool = ServerPool()
    try:
        for name, path in families.items():
            pool.start(name, path, "stateless", num_processes=args.processes, env_kwargs=json.loads(args.env_kwargs))
        if args.check:
            for name in families:
                out = pool.get(name).rollout({}, [])
                print(f"env host: family {name} answered with keys {sorted(out)}")
            return 0
        import uvicorn

        uvicorn.run(http_app(pool), host=args.host, port=args.port, log_level="warning")
        return 0
    finally:
        pool.close()


if __name__ == "__main__":
    raise SystemExit(main())
