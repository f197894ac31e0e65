"""Learner -> rollout-engine weight synchronisation.

The reference gathers the whole model on every learner, clones each tensor on rank 0 and sends 291
NCCL broadcasts to the vLLM workers, which then re-fuse QKV and gate/up on their side
(``open_instruct/vllm_utils.py:1383-1480``).  Here learner and engine share ONE flat fused layout, so a
sync is a slice copy: every learner rank pushes its 1/world slice of the bf16 working copy straight
into every engine's parameter buffer with one kernel (one read, one NVLink store per engine;
``ops/csrc/zero_comm.cu:multi_push_kernel``).  Engine buffers living in other processes are mapped
through CUDA IPC (``EngineWorker.weight_buffer_ipc`` / ``LearnerWorker.connect_engines``); in a shared
process the destination is an ordinary tensor.
"""

from __future__ import annotations

import ctypes
import time

import torch

from ..ops import lib
from ..ops.lib import ptr, stream_ptr

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
lib._SIGNATURES["b200_multi_push"] = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), _I, _L, _L, _I, _P]


_peer_ok: set[tuple[int, int]] = set()


def ensure_peer_access(dev: int, peer: int) -> None:
    """Kernels on ``dev`` may then store into ``peer``'s memory.  Idempotent; raises if the GPUs are not connected."""
    if dev == peer or (dev, peer) in _peer_ok:
        return
    so = lib.load_ops()
    so.b200_enable_peer_access.argtypes = [_I, _I]
    so.b200_enable_peer_access.restype = _I
    rc = so.b200_enable_peer_access(dev, peer)
    if rc:
        raise lib.KernelError(f"cannot enable peer access from GPU {dev} to GPU {peer} (code {rc})")
    _peer_ok.add((dev, peer))


def push_slice(src: torch.Tensor, dsts: list[torch.Tensor], lo: int, hi: int) -> None:
    """``dst[lo:hi] = bf16(src[lo:hi])`` for every destination (CUDA: one kernel for all of them)."""
    if hi <= lo or not dsts:
        return
    if src.is_cuda and all(d.is_cuda and d.dtype == torch.bfloat16 for d in dsts) and lo % 8 == 0 and len(dsts) <= 8:
        so = lib.load_ops()
        for d in dsts:
            ensure_peer_access(src.device.index, d.device.index)
        fn = so.b200_multi_push
        fn.argtypes = [_P, ctypes.POINTER(ctypes.c_void_p), _I, _L, _L, _I, _P]
        fn.restype = _I
        arr = (ctypes.c_void_p * 8)()
        for i, d in enumerate(dsts):
            arr[i] = d.data_ptr()
        rc = fn(ptr(src), arr, len(dsts), lo, hi - lo, int(src.dtype == torch.float32), stream_ptr())
        lib.launch_count += 1
        if rc:
            raise lib.KernelError(f"b200_multi_push failed with code {rc}")
        return
    with torch.no_grad():
        for d in dsts:
            d[lo:hi].copy_(src[lo:hi].to(d.dtype), non_blocking=True)


def sync_in_process(learner_flat: torch.Tensor, engines: list, model_step: int, total: int) -> float:
    """Single-process mode: push the whole model into every engine and stamp the new version."""
    t0 = time.perf_counter()
    views = [e.engine.model.flat.detach() for e in engines]
    for e in engines:
        e.lock.acquire()
    try:
        push_slice(learner_flat.detach(), views, 0, total)
        if learner_flat.is_cuda:
            torch.cuda.synchronize(learner_flat.device)
        for e in engines:
            e.engine.model_step = model_step
    finally:
        for e in engines:
            e.lock.release()
    return time.perf_counter() - t0
