"""TransferQueue: the store through which finished trajectories travel from the agent loop to the trainer.

The role of the upstream ``TransferQueue`` (a controller plus ``num_data_storage_units`` storage actors,
``pear/configs/base.yaml:107-112``): trajectories are written field by field under a key (``<prompt uid>/<session>``),
a key becomes visible to readers only once it is sealed, storage is spread over a fixed number of units by key hash,
and a snapshot writes ONE FILE PER STORAGE UNIT (so 32 writers work in parallel and a snapshot only loads into the same
number of units). A key that was being written when the snapshot was taken (unsealed) is dropped at load time
(upstream ``trainer.py:159-244`` "drops half-written keys").
"""

from __future__ import annotations

import os
import pickle
import threading
import zlib
from dataclasses import dataclass, field
from typing import Any, Iterable, Optional

from ..utils.files import atomic_write


@dataclass
class _Entry:
    fields: dict[str, Any] = field(default_factory=dict)
    sealed: bool = False
    meta: dict[str, Any] = field(default_factory=dict)


class StorageUnit:
    def __init__(self, index: int):
        self.index = index
        self.entries: dict[str, _Entry] = {}
        self.lock = threading.Lock()

    def put(self, key: str, name: str, value: Any) -> None:
        with self.lock:
            self.entries.setdefault(key, _Entry()).fields[name] = value

    def seal(self, key: str, meta: Optional[dict] = None) -> None:
        with self.lock:
            e = self.entries.setdefault(key, _Entry())
            e.sealed = True
            if meta:
                e.meta.update(meta)

    def get(self, key: str) -> Optional[_Entry]:
        with self.lock:
            e = self.entries.get(key)
            return e if (e is not None and e.sealed) else None

    def pop(self, key: str) -> None:
        with self.lock:
            self.entries.pop(key, None)

    def snapshot(self, path: str) -> None:
        with self.lock:
            data = {k: (e.fields, e.sealed, e.meta) for k, e in self.entries.items()}
        atomic_write(path, pickle.dumps(data, protocol=pickle.HIGHEST_PROTOCOL), binary=True)

    def restore(self, path: str) -> int:
        with open(path, "rb") as f:
            data = pickle.load(f)
        dropped = 0
        with self.lock:
            self.entries.clear()
            for k, (fields, sealed, meta) in data.items():
                if not sealed:
                    dropped += 1  # torn write: the session will be re-run
                    continue
                self.entries[k] = _Entry(fields, True, meta)
        return dropped


class TransferQueue:
    def __init__(self, num_data_storage_units: int = 32):
        self.units = [StorageUnit(i) for i in range(num_data_storage_units)]

    def _unit(self, key: str) -> StorageUnit:
        return self.units[zlib.crc32(key.encode()) % len(self.units)]

    # -- writers (agent loop) ---------------------------------------------------------------------------------------
    def put(self, key: str, **fields: Any) -> None:
        u = self._unit(key)
        for name, value in fields.items():
            u.put(key, name, value)

    def seal(self, key: str, **meta: Any) -> None:
        self._unit(key).seal(key, meta)

    def put_trajectory(self, key: str, fields: dict[str, Any], **meta: Any) -> None:
        self.put(key, **fields)
        self.seal(key, **meta)

    # -- readers (trainer) ------------------------------------------------------------------------------------------
    def get(self, key: str) -> Optional[dict[str, Any]]:
        e = self._unit(key).get(key)
        return None if e is None else dict(e.fields, **{"__meta__": dict(e.meta)})

    def has(self, key: str) -> bool:
        return self._unit(key).get(key) is not None

    def keys(self, prefix: str = "", sealed_only: bool = True) -> list[str]:
        out = []
        for u in self.units:
            with u.lock:
                out += [k for k, e in u.entries.items() if k.startswith(prefix) and (e.sealed or not sealed_only)]
        return sorted(out)

    def clear(self, keys: Iterable[str]) -> None:
        for k in keys:
            self._unit(k).pop(k)

    def clear_prefix(self, prefix: str) -> int:
        ks = self.keys(prefix, sealed_only=False)
        self.clear(ks)
        return len(ks)

    # -- snapshot ---------------------------------------------------------------------------------------------------
    def snapshot(self, directory: str) -> None:
        os.makedirs(directory, exist_ok=True)
        threads = [threading.Thread(target=u.snapshot, args=(os.path.join(directory, f"unit_{u.index:03d}.pkl"),)) for u in self.units]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        atomic_write(os.path.join(directory, "units.txt"), str(len(self.units)))

    def restore(self, directory: str) -> int:
        """Returns the number of half-written keys that were dropped."""
        with open(os.path.join(directory, "units.txt")) as f:
            n = int(f.read().strip())
        if n != len(self.units):
            raise ValueError(f"snapshot of {n} storage units cannot load into {len(self.units)}")
        return sum(u.restore(os.path.join(directory, f"unit_{u.index:03d}.pkl")) for u in self.units)

    def close(self) -> None:
        for u in self.units:
            with u.lock:
                u.entries.clear()
