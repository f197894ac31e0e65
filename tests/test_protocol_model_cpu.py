"""Host-side model of the device protocols: CPU threads stand in for ranks, shared Python lists for symmetric memory.

1. Epoch barrier through per-rank signal pads (``symm_barrier_kernel``): nobody passes barrier ``e`` before everyone arrived.
2. One-shot all-reduce with two alternating exchange buffers and a flag handshake per call (``tp_allreduce_norm_kernel``):
   a rank may overwrite buffer ``k`` for call ``n + 2`` only after every peer finished reading call ``n`` - the model checks
   that the values a reader sees always belong to the call it is reducing, under random delays.
"""

import random
import threading
import time


def test_epoch_barrier_model():
    world, rounds = 4, 200
    pads = [[0] * world for _ in range(world)]  # pads[r][p]: slot of peer p in rank r's pad
    arrived = [0] * world
    errors = []

    def rank_fn(r):
        rng = random.Random(r)
        for e in range(1, rounds + 1):
            if rng.random() < 0.2:
                time.sleep(rng.random() * 1e-4)
            arrived[r] = e
            for p in range(world):
                pads[p][r] = e          # publish my arrival in every peer's pad
            for p in range(world):
                while pads[r][p] - e < 0:  # wait for every peer's flag in MY pad (wrap-safe comparison in the kernel)
                    time.sleep(0)
            if min(arrived) < e:
                errors.append((r, e, list(arrived)))

    ts = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert not errors and all(a == rounds for a in arrived)


def test_double_buffered_one_shot_allreduce_model():
    world, calls = 3, 300
    bufs = [[[None] * 1 for _ in range(2)] for _ in range(world)]  # bufs[rank][parity][0] = (call id, value)
    flags = [[0] * world for _ in range(world)]
    errors, results = [], [[None] * calls for _ in range(world)]

    def rank_fn(r):
        rng = random.Random(100 + r)
        for n in range(calls):
            par = n & 1
            if rng.random() < 0.3:
                time.sleep(rng.random() * 1e-4)
            bufs[r][par][0] = (n, (r + 1) * (n + 1))   # the "GEMM" writes this rank's partial for call n
            for p in range(world):
                flags[p][r] = n + 1                     # kernel start: signal epoch n + 1 to every peer
            total = 0
            for p in range(world):
                while flags[r][p] < n + 1:
                    time.sleep(0)
                cid, val = bufs[p][par][0]              # peer load
                if cid != n:
                    errors.append((r, n, p, cid))
                total += val
            results[r][n] = total

    ts = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(120) for t in ts]
    assert not errors, errors[:5]
    for n in range(calls):
        want = sum((p + 1) * (n + 1) for p in range(world))
        assert all(results[r][n] == want for r in range(world))
