"""Pool of environment instances shared by the rollout workers: ``acquire`` hands out a free
instance (waiting up to a timeout), ``release`` returns it (``open_instruct/environments/pool.py:12-58``)."""

from __future__ import annotations

import queue
import threading

ACQUIRE_TIMEOUT_S = 7200


class EnvironmentPool:
    def __init__(self, factory, pool_size: int):
        self._free: queue.Queue = queue.Queue()
        self._all = [factory() for _ in range(pool_size)]
        for e in self._all:
            self._free.put(e)
        self._lock = threading.Lock()
        self.in_use = 0

    def acquire(self, timeout: float = ACQUIRE_TIMEOUT_S):
        try:
            env = self._free.get(timeout=timeout)
        except queue.Empty:
            raise TimeoutError(f"no free environment after {timeout}s (pool of {len(self._all)})") from None
        with self._lock:
            self.in_use += 1
        return env

    def release(self, env) -> None:
        with self._lock:
            self.in_use -= 1
        self._free.put(env)

    def size(self) -> int:
        return len(self._all)

    def tool_definitions(self) -> list[dict]:
        return self._all[0].get_tool_definitions() if self._all else []

    def close(self) -> None:
        for e in self._all:
            e.close()
