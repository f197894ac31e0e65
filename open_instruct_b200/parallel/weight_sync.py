"""Learner -> rollout-engine weight synchronisation.

The reference gathers the whole model on every learner, clones each tensor on rank 0 and sends 291
NCCL broadcasts to the vLLM workers, which then re-fuse QKV and gate/up on their side
(``open_instruct/vllm_utils.py:1383-1480``).  Here learner and engine share ONE flat fused layout, so a
sync is a slice copy: every learner rank pushes its 1/world slice of the bf16 working copy straight
into every engine's parameter buffer with one kernel (one read, one NVLink store per engine;
``ops/csrc/zero_comm.cu:multi_push_kernel``).  Engine buffers living in other processes are mapped
through CUDA IPC (``export_buffer`` in the engine process, ``import_buffer`` in the learner process, which opens
the handle with the learner's GPU current so that the mapping lives in the address space its kernels use); in a
shared process the destination is an ordinary tensor.
"""

from __future__ import annotations

import ctypes
import time

import torch

from ..ops import lib
from ..ops.lib import ptr, stream_ptr

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
lib._SIGNATURES["b200_multi_push"] = [_P, ctypes.POINTER(ctypes.c_void_p), _I, _L, _L, _I, _P]


class PeerBuffer:
    """A bf16 buffer of another process, mapped into this one for kernels of GPU ``mapped_for``."""

    is_cuda, dtype = True, torch.bfloat16

    def __init__(self, base: int, offset: int, numel: int, owner_device: int, mapped_for: int):
        self.base, self.offset, self._numel, self.owner_device, self.mapped_for = base, offset, numel, owner_device, mapped_for

    def data_ptr(self) -> int:
        return self.base + self.offset

    def numel(self) -> int:
        return self._numel

    def close(self) -> None:
        if self.base:
            so = lib.load_ops()
            so.b200_ipc_close.argtypes = [_I, _P]
            so.b200_ipc_close.restype = _I
            so.b200_ipc_close(self.mapped_for, self.base)
            self.base = 0


def export_buffer(t: torch.Tensor) -> dict:
    """Picklable description of a CUDA tensor's memory for ``import_buffer`` in another process."""
    so = lib.load_ops()
    so.b200_ipc_export.argtypes = [_P, ctypes.c_char_p, ctypes.POINTER(_L), ctypes.POINTER(_L)]
    so.b200_ipc_export.restype = _I
    handle = ctypes.create_string_buffer(64)
    off, size = _L(0), _L(0)
    with torch.cuda.device(t.device):
        rc = so.b200_ipc_export(ptr(t), handle, ctypes.byref(off), ctypes.byref(size))
    if rc:
        raise lib.KernelError(f"cannot export buffer for inter-process sharing (code {rc})")
    return {"handle": handle.raw, "offset": off.value, "numel": t.numel(), "dtype": str(t.dtype), "device": t.device.index}


def import_buffer(desc: dict, device_index: int) -> PeerBuffer:
    """Map an exported buffer for kernels that run on ``device_index`` of this process."""
    if desc["dtype"] != "torch.bfloat16":
        raise ValueError("weight buffers are shared as bf16")
    so = lib.load_ops()
    so.b200_ipc_open.argtypes = [_I, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    so.b200_ipc_open.restype = _I
    base = ctypes.c_void_p(0)
    rc = so.b200_ipc_open(device_index, desc["handle"], ctypes.byref(base))
    if rc or not base.value:
        raise lib.KernelError(f"cannot map a peer process's buffer on GPU {device_index} (code {rc})")
    return PeerBuffer(base.value, desc["offset"], desc["numel"], desc["device"], device_index)


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


def push_slice(src: torch.Tensor, dsts: list[torch.Tensor], lo: int, hi: int, src_offset: int | None = None) -> None:
    """``dst[lo:hi] = bf16(src[lo:hi])`` for every destination (CUDA: one kernel for all of them).  With ``src_offset`` the
    source range starts there instead of at ``lo`` (a rank that holds only its slice of the parameters pushes it to its
    place in the engines' full buffers)."""
    if hi <= lo or not dsts:
        return
    so_ = lo if src_offset is None else src_offset
    if so_ % 8:
        raise ValueError("source offset must be a multiple of 8 elements")
    if any(isinstance(d, PeerBuffer) for d in dsts) and not (src.is_cuda and lo % 8 == 0 and len(dsts) <= 8):
        raise ValueError("buffers of other processes can only be written by the push kernel (CUDA source, offset multiple of 8, <= 8 engines)")
    if src.is_cuda and all(d.is_cuda and d.dtype == torch.bfloat16 for d in dsts) and lo % 8 == 0 and len(dsts) <= 8:
        so = lib.load_ops()
        for d in dsts:
            if hi > d.numel():
                raise ValueError("destination buffer is smaller than the pushed range")
            if isinstance(d, PeerBuffer):
                if d.mapped_for != src.device.index:
                    raise ValueError(f"buffer was mapped for GPU {d.mapped_for} but the push runs on GPU {src.device.index}")
            else:
                ensure_peer_access(src.device.index, d.device.index)
        fn = so.b200_multi_push
        fn.argtypes = [_P, ctypes.POINTER(ctypes.c_void_p), _I, _L, _L, _I, _P]
        fn.restype = _I
        arr = (ctypes.c_void_p * 8)()
        for i, d in enumerate(dsts):
            arr[i] = d.data_ptr()
        with torch.cuda.device(src.device):  # the launch goes to the source GPU whatever this thread's current device is
            # the kernel indexes source and destinations with the same offset: shift the source base instead
            rc = fn(ptr(src) + (so_ - lo) * src.element_size(), arr, len(dsts), lo, hi - lo, int(src.dtype == torch.float32), stream_ptr())
        lib.launch_count += 1
        if rc:
            raise lib.KernelError(f"b200_multi_push failed with code {rc}")
        return
    with torch.no_grad():
        for d in dsts:
            d[lo:hi].copy_(src[so_:so_ + hi - lo].to(d.dtype), non_blocking=True)


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
