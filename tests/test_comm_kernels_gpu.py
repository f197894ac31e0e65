"""The data paths of the multi-GPU kernels on ONE GPU: every "peer" pointer is another buffer of the same device.

The kernels that move gradients, parameters and weights between GPUs take a table of peer pointers; nothing in them
depends on the pointers belonging to different devices.  Pointing the table at local buffers checks their index
arithmetic, tails and numerics against plain PyTorch on a single-GPU machine.  (The flag exchanges between ranks are
not part of this: kernels that wait on one another never run as separate launches on one GPU; those are covered by
the 2-GPU workers and by the CPU protocol model.)
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptrs(tensors):
    arr = (ctypes.c_void_p * 8)()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


@pytest.fixture(scope="module")
def symm_mod():
    from open_instruct_b200.ops import lib

    if not lib.available():
        pytest.skip("needs a B200")
    from open_instruct_b200.parallel import symm, weight_sync, zero3_peer  # noqa: F401 - register the C signatures

    return lib


@pytest.mark.parametrize("world,n,lo", [(2, 4096, 0), (4, 1 << 20, 1024), (8, 333 * 4, 128), (3, 4, 0)])
def test_reduce_range_virtual_peers(symm_mod, world, n, lo):
    lib = symm_mod
    torch.manual_seed(world)
    bufs = [torch.randn(lo + n + 64, device="cuda") for _ in range(world)]
    out = torch.full((n + 8,), 7.0, device="cuda")
    sq = torch.zeros(1, device="cuda")
    for ctas in (0, 3):
        out.fill_(7.0)
        sq.zero_()
        lib.call("b200_zero_reduce_range", _ptrs(bufs), None, world, lo, n, out.data_ptr(), sq.data_ptr(), 0, ctas,
                 lib.stream_ptr())
        want = torch.stack([b[lo:lo + n] for b in bufs]).double().sum(0)
        torch.testing.assert_close(out[:n].double(), want, atol=1e-5, rtol=1e-5)
        assert torch.all(out[n:] == 7.0)  # nothing written past the range
        torch.testing.assert_close(sq.double(), want.float().double().pow(2).sum().reshape(1), rtol=1e-4, atol=1e-4)
    lib.check_status()


def test_reduce_scatter_sum_is_rank_order_deterministic(symm_mod):
    lib = symm_mod
    bufs = [torch.randn(1 << 16, device="cuda") * 10 ** (i - 2) for i in range(5)]
    outs = []
    for _ in range(2):
        out, sq = torch.empty(1 << 16, device="cuda"), torch.zeros(1, device="cuda")
        lib.call("b200_zero_reduce_range", _ptrs(bufs), None, 5, 0, 1 << 16, out.data_ptr(), sq.data_ptr(), 0, 0, lib.stream_ptr())
        outs.append(out)
    acc = torch.zeros_like(bufs[0])
    for b in bufs:  # the kernel adds in rank order starting from zero
        acc = acc + b
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], acc)


@pytest.mark.parametrize("world", [1, 3, 8])
def test_adamw_allgather_virtual_peers(symm_mod, world):
    from open_instruct_b200.ops import ref

    lib = symm_mod
    n, goff = 8 * 1000, 64
    torch.manual_seed(0)
    master = torch.randn(n, device="cuda")
    m, v = torch.rand(n, device="cuda") * 0.1, torch.rand(n, device="cuda") * 0.01
    g = torch.randn(n, device="cuda")
    gs = torch.tensor([0.5], device="cuda")
    params = [torch.zeros(goff + n + 16, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    M, m2, v2 = master.clone(), m.clone(), v.clone()
    ref.adamw_step(M, m2, v2, g.clone(), 1e-2, 0.9, 0.999, 1e-8, 0.1, 3, gscale=gs)
    lib.call("b200_zero_adamw_allgather", master.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), _ptrs(params), None, world,
             goff, n, gs.data_ptr(), 1e-2, 0.9, 0.999, 1e-8, 0.1, 3, 0, lib.stream_ptr())
    torch.testing.assert_close(master, M, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(m, m2, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(v, v2, atol=1e-7, rtol=1e-5)
    for p in params:
        assert torch.equal(p[goff:goff + n], master.bfloat16())
        assert torch.all(p[:goff] == 0) and torch.all(p[goff + n:] == 0)
    lib.check_status()


@pytest.mark.parametrize("src_f32", [0, 1])
def test_multi_push_virtual_peers(symm_mod, src_f32):
    lib = symm_mod
    n, off = 8 * 4097 + 5, 16
    src = torch.randn(off + n, device="cuda")
    if not src_f32:
        src = src.bfloat16()
    dsts = [torch.zeros(off + n + 8, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    lib.call("b200_multi_push", src.data_ptr(), _ptrs(dsts), 3, off, n, src_f32,
             lib.stream_ptr())
    for d in dsts:
        assert torch.equal(d[off:off + n], src[off:off + n].bfloat16())
        assert torch.all(d[:off] == 0) and torch.all(d[off + n:] == 0)


def test_allgather_pull_and_reduce_scatter_add_virtual_peers(symm_mod):
    lib = symm_mod
    world, n, soff = 4, 8 * 513, 24
    shards = [torch.randn(soff + n, device="cuda").bfloat16() for _ in range(world)]
    out = torch.zeros(world * n, dtype=torch.bfloat16, device="cuda")
    lib.call("b200_allgather_pull", _ptrs(shards), world, soff, n, out.data_ptr(), 4, lib.stream_ptr())
    assert torch.equal(out, torch.cat([s[soff:] for s in shards]))
    ws = [torch.randn(1024 + 4 * 777, device="cuda") for _ in range(world)]
    acc = torch.randn(4 * 777, device="cuda")
    want = acc.double() + torch.stack([w[1024:] for w in ws]).double().sum(0)
    lib.call("b200_reduce_scatter_add", _ptrs(ws), None, world, 1024, 4 * 777, acc.data_ptr(), 2, lib.stream_ptr())
    torch.testing.assert_close(acc.double(), want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("src_f32", [False, True])
def test_tp_push_writes_every_rank_its_shard(symm_mod, src_f32):
    """The tensor-parallel weight push (2 engines x TP 2, four destination buffers on this GPU) against ``shard_flat``: every
    learner slice of the full layout lands in its place of every rank's shard layout, nothing else is touched."""
    from open_instruct_b200.models.spec import ParamLayout, get_spec
    from open_instruct_b200.parallel.tp import local_spec, shard_flat
    from open_instruct_b200.parallel.weight_sync import push_tp, tp_push_plan

    spec = get_spec("tiny128-tp").replace(qk_norm=True, attention_bias=True, model_type="qwen3")
    tp, engines, world = 2, 2, 3
    full, loc = ParamLayout(spec), ParamLayout(local_spec(spec, tp))
    src = torch.randn(full.total, device="cuda")
    src16 = src.bfloat16()
    dsts = [torch.full((loc.total + 64,), 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(engines * tp)]
    per = (-(-full.total // world) + 1023) // 1024 * 1024
    for r in range(world):
        lo, hi = min(full.total, r * per), min(full.total, (r + 1) * per)
        plan = tp_push_plan(spec, tp, lo, hi, n_engines=engines)
        dev = torch.from_numpy(plan.view("u1").copy()).cuda()
        push_tp(src if src_f32 else src16, dsts, dev, len(plan))
    torch.cuda.synchronize()
    for e in range(engines):
        for r in range(tp):
            want = shard_flat(src16, spec, r, tp)
            got = dsts[e * tp + r]
            for name, v in loc.views(got[: loc.total]).items():
                assert torch.equal(v, loc.views(want)[name]), (e, r, name)
            assert torch.all(got[loc.total:] == 9.0)
