"""File helpers: advisory file lock, atomic writes (upstream ``pear/utils``: ``FileLock``, atomic write)."""

from __future__ import annotations

import fcntl
import os
import tempfile


class FileLock:
    """``with FileLock(path):`` holds an exclusive advisory lock on ``path`` (created if missing)."""

    def __init__(self, path: str):
        self.path, self.fd = path, None

    def __enter__(self) -> "FileLock":
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        self.fd = os.open(self.path, os.O_CREAT | os.O_RDWR, 0o644)
        fcntl.flock(self.fd, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc) -> None:
        fcntl.flock(self.fd, fcntl.LOCK_UN)
        os.close(self.fd)
        self.fd = None


def atomic_write(path: str, data, binary: bool = False) -> None:
    """Write to a temporary sibling, fsync, rename: readers see the old or the new file, never a torn one."""
    d = os.path.dirname(os.path.abspath(path))
    os.makedirs(d, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=d, prefix=".tmp_" + os.path.basename(path))
    try:
        with os.fdopen(fd, "wb" if binary else "w") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def append_jsonl(path: str, record: dict) -> None:
    """Append one JSON line under the file's lock (several processes may log to the same file)."""
    import json

    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with FileLock(path + ".lock"):
        with open(path, "a") as f:
            f.write(json.dumps(record, default=str) + "\n")
