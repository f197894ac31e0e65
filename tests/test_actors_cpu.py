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

    def twice(self, t):
        return {"out": t * 2, "n": t.numel()}


class DiesInInit:
    def __init__(self):
        import os

        os._exit(9)  # what the kernel's out-of-memory killer or a native crash looks like from outside


def test_an_actor_that_dies_while_starting_is_reported_at_once():
    from open_instruct_b200.actors import ray_compat as ray

    t0 = time.time()
    with pytest.raises(ray.ActorError, match="died while starting"):
        ray.remote(DiesInInit).remote()
    assert time.time() - t0 < 30


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


def test_bulk_payloads_go_through_shared_memory():
    """Tensors and arrays above the threshold leave the pickle stream and cross in one shared-memory segment that the receiver
    unlinks; small messages stay plain pickles; values, dtypes (bf16 included), shapes and non-contiguous views survive."""
    import glob
    import pickle

    import numpy as np
    import torch

    from open_instruct_b200.actors import ray_compat as rc

    small = {"a": torch.arange(10), "s": "text", "n": np.arange(5)}
    raw = rc._dumps(small)
    assert not raw.startswith(rc._SHM_MAGIC)
    back = rc._loads(raw)
    assert torch.equal(back["a"], small["a"]) and back["s"] == "text" and (back["n"] == small["n"]).all()
    big = {"ids": torch.randint(0, 1000, (64, 4096)), "w": torch.randn(300, 700).bfloat16(), "view": torch.randn(512, 512)[:, ::2],
           "arr": np.random.rand(200_000), "nested": [torch.ones(3), ("x", torch.full((70_000,), 2.5))], "scalar": 7}
    before = set(glob.glob("/dev/shm/psm_*"))
    raw = rc._dumps(big)
    assert raw.startswith(rc._SHM_MAGIC) and len(raw) < 20_000          # only names, layout and the pickle skeleton travel on the socket
    name, layout, _ = pickle.loads(raw[len(rc._SHM_MAGIC):])
    assert len(set(glob.glob("/dev/shm/psm_*")) - before) == 1 and sum(n for _, n in layout) > 3_000_000
    back = rc._loads(raw)
    assert set(glob.glob("/dev/shm/psm_*")) - before == set()                 # the receiver removed the segment
    assert torch.equal(back["ids"], big["ids"]) and back["w"].dtype == torch.bfloat16 and torch.equal(back["w"], big["w"])
    assert torch.equal(back["view"], big["view"]) and back["view"].is_contiguous()
    assert (back["arr"] == big["arr"]).all() and torch.equal(back["nested"][1][1], big["nested"][1][1]) and back["scalar"] == 7
    back["ids"][0, 0] = -1                                                     # received tensors own writable memory
    assert back["ids"][0, 0] == -1


def test_actor_call_with_a_bulk_argument_and_result():
    import torch

    from open_instruct_b200.actors import ray_compat as rc

    h = rc.remote(Counter).remote()
    try:
        x = torch.randn(1024, 1024)   # 4 MiB each way
        res = rc.get(h.twice.remote(x))
        assert res["n"] == x.numel() and torch.equal(res["out"], x * 2)
    finally:
        rc.kill(h)
