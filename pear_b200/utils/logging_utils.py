"""Logger with its own handler (it does not depend on the root logger's configuration) and the one-line structured
events the monitor parses: ``phase <name>`` per timed phase, ``EPISODE_END {...}``, ``PARSE_FAILURE``,
``TRAJECTORY_RESTART`` (upstream ``pear/utils/logging_utils.py:6-17``, ``3rdparty/verl/patches/0013-*``)."""

from __future__ import annotations

import contextlib
import json
import logging
import sys
import time


def get_logger(name: str = "pear_b200", level: int = logging.INFO, stream=None) -> logging.Logger:
    log = logging.getLogger(name)
    if not any(getattr(h, "_pear", False) for h in log.handlers):
        h = logging.StreamHandler(stream or sys.stderr)
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))
        h._pear = True
        log.addHandler(h)
        log.propagate = False
    log.setLevel(level)
    return log


def add_file_handler(log: logging.Logger, path: str) -> None:
    h = logging.FileHandler(path)
    h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))
    h._pear = True
    log.addHandler(h)


def event(log: logging.Logger, name: str, **fields) -> None:
    log.info("%s %s", name, json.dumps(fields, sort_keys=True, default=str))


@contextlib.contextmanager
def phase(log: logging.Logger, name: str, timings: dict | None = None):
    """Times a phase, logs ``phase <name> <seconds>`` and records ``timing_s/<name>``."""
    t0 = time.time()
    try:
        yield
    finally:
        dt = time.time() - t0
        log.info("phase %s %.3f", name, dt)
        if timings is not None:
            timings[f"timing_s/{name}"] = timings.get(f"timing_s/{name}", 0.0) + dt
