"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory when they need this op (they
run inside someone else's memory pool, or were handed fixed buffers), so this variant keeps its
scratch inside the library.  It must give the same numbers as the ordinary entry point, on
repeated calls, whether or not other kernels of the library ran before it in the process.
This file is collected last on purpose.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind():
    from open_instruct_b200.ops import lib

    so = lib.load_ops()
    fn = so.b200_rmsnorm_bwd_noalloc
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, P, P, P, P, I, I, P]
    fn.restype = I
    so.b200_rmsnorm_bwd_noalloc_max_d.restype = I
    so.b200_rmsnorm_bwd_noalloc_max_d.argtypes = []
    return so, fn


def test_noalloc_matches_regular_entry_twice():
    from open_instruct_b200.ops import fused

    so, fn = _bind()
    stream = torch.cuda.current_stream().cuda_stream
    # the first call on a device does the one-time set-up (symbol address, kernel attribute, lazy module load): make it
    # here, so that the calls measured below are ordinary ones
    z, z_out, ones = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16), torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16), torch.ones(8, device="cuda")
    assert fn(z.data_ptr(), z.data_ptr(), ones.data_ptr(), z.data_ptr(), None, z_out.data_ptr(), None, 8, 64, stream) == 0
    torch.cuda.synchronize()
    for call, (T, D) in enumerate([(777, 4096), (300, 1024)]):
        g = torch.Generator(device="cuda").manual_seed(call)
        h = torch.randn(T, D, device="cuda", generator=g).bfloat16()
        w = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
        dy = torch.randn(T, D, device="cuda", generator=g).bfloat16()
        dres = torch.randn(T, D, device="cuda", generator=g).bfloat16()
        rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-5)
        dw_ref = torch.zeros(D, device="cuda")
        dx_ref = fused.rmsnorm_bwd(h, w, rstd, dy, dres, dw_ref)
        dx = torch.empty_like(h)
        dw = torch.zeros(D, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()  # the driver's view: also sees a cudaMalloc made inside the library
        rc = fn(h.data_ptr(), w.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dres.data_ptr(), dx.data_ptr(),
                dw.data_ptr(), T, D, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated during the call"
        assert torch.equal(dx, dx_ref)
        assert ((dw - dw_ref).abs().max() / dw_ref.abs().max()).item() < 1e-5


def test_noalloc_rejects_oversize():
    so, fn = _bind()
    max_d = so.b200_rmsnorm_bwd_noalloc_max_d()
    D = max_d + 8
    x = torch.zeros(1, D, device="cuda", dtype=torch.bfloat16)
    r = torch.ones(1, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), r.data_ptr(), x.data_ptr(), None, x.data_ptr(), None, 1, D,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -3
