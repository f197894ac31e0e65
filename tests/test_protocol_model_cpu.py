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


def test_sharded_gradient_workspace_model():
    """Per-layer gradient reduction of the parameter-sharded learner (``parallel/zero3.py`` with the peer transport): two
    workspaces per rank alternate between layers; for layer ``i`` every rank runs, on its communication "stream",
    barrier - read every peer's workspace ``i & 1`` - barrier, and its compute "stream" may overwrite a workspace only after
    the communication stream finished the reduction that last used it.  The model gives each rank a compute thread and a
    communication thread and checks that a reader always sees the layer it is reducing."""
    world, layers = 3, 120
    ws = [[None, None] for _ in range(world)]            # ws[rank][slot] = layer id whose gradients it holds
    pads = [[0] * world for _ in range(world)]
    written = [[threading.Event() for _ in range(layers)] for _ in range(world)]   # compute -> comm: layer i is written
    reduced = [[threading.Event() for _ in range(layers)] for _ in range(world)]   # comm -> compute: reduction i is over
    errors = []

    def barrier(r, epoch):
        for p in range(world):
            pads[p][r] = epoch
        for p in range(world):
            while pads[r][p] - epoch < 0:
                time.sleep(0)

    def compute(r):
        rng = random.Random(r)
        for i in range(layers):
            if i >= 2:
                reduced[r][i - 2].wait()                  # the event recorded after the closing barrier of reduction i - 2
            if rng.random() < 0.3:
                time.sleep(rng.random() * 2e-4)
            ws[r][i & 1] = i                              # the weight-gradient GEMMs overwrite the workspace
            written[r][i].set()

    def comm(r):
        rng = random.Random(1000 + r)
        epoch = 0
        for i in range(layers):
            written[r][i].wait()                          # stream order: after this rank's backward of layer i
            epoch += 1
            barrier(r, epoch)                             # every rank has written layer i
            for p in range(world):
                if rng.random() < 0.2:
                    time.sleep(rng.random() * 1e-4)
                if ws[p][i & 1] != i:                     # peer load
                    errors.append((r, i, p, ws[p][i & 1]))
            epoch += 1
            barrier(r, epoch)                             # every rank has finished reading
            reduced[r][i].set()

    ts = [threading.Thread(target=f, args=(r,)) for r in range(world) for f in (compute, comm)]
    [t.start() for t in ts]
    [t.join(120) for t in ts]
    assert not any(t.is_alive() for t in ts)
    assert not errors, errors[:5]
