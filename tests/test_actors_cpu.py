"""Actor runtime: process actors, futures, named actors, cross-process queues, error propagation."""

import time

import pytest


class Counter:
    def __init__(self, start=0):
        self.v = start

    def add(self, n):
        self.v += n
        return self.v

    def slow(self, t):
        time.sleep(t)
        return "done"

    def boom(self):
        raise ValueError("bad thing")

    def use_queue(self, q, item):
        q.put(item)
        return q.qsize()


def test_actor_calls_and_errors():
    from open_instruct_b200.actors import ray_compat as ray

    try:
        C = ray.remote(Counter)
        a = C.options(name="ctr").remote(5)
        assert ray.get(a.add.remote(3)) == 8
        assert max(ray.get([a.add.remote(1), a.add.remote(1)])) == 10  # concurrent calls may finish in either order
        assert ray.get(ray.get_actor("ctr").add.remote(0)) == 10
        t0 = time.time()
        refs = [a.slow.remote(0.3) for _ in range(4)]  # threaded actor: calls overlap
        assert ray.get(refs) == ["done"] * 4 and time.time() - t0 < 1.0
        done, pending = ray.wait([a.slow.remote(0.5)], num_returns=1, timeout=0.05)
        assert not done and len(pending) == 1
        with pytest.raises(ray.ActorError, match="bad thing"):
            ray.get(a.boom.remote())
        q = ray.Queue(maxsize=2)
        assert ray.get(a.use_queue.remote(q, "x")) == 1  # queue handle travels to another process
        assert q.get(timeout=1) == "x"
        with pytest.raises(ray.Empty):
            q.get_nowait()
        q.put(1); q.put(2)
        with pytest.raises(ray.Full):
            q.put_nowait(3)
        ray.kill(a)
        with pytest.raises(ray.ActorError):
            ray.get(a.add.remote(1), timeout=5)
    finally:
        ray.shutdown()
