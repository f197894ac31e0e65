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


# ------------------------------------------------------------------------------------------------ tensor-parallel engines
lib._SIGNATURES["b200_tp_push"] = [_P, ctypes.POINTER(ctypes.c_void_p), _I, _P, _I, _I, _P]
TILE_DTYPE = [("src", "<i8"), ("dst", "<i8"), ("src_stride", "<i8"), ("dst_stride", "<i8"), ("rows", "<i4"), ("row_len", "<i4"), ("mask", "<u4"), ("pad", "<i4")]


def _tp_pieces(spec, tp: int):
    """Every piece of the full flat layout with its place in the tensor-parallel ranks' local layouts:
    ``(src_off, rows, row_len, src_stride, dst_off, dst_stride, rank or -1 for all ranks)`` in elements.  This is the
    re-layout ``parallel.tp.shard_flat`` performs, written as 2-D copies (what vLLM's ``load_weights`` does per worker in
    the reference, ``open_instruct/vllm_utils.py:1383-1480``)."""
    from ..models.spec import ParamLayout
    from .tp import local_spec

    ls = local_spec(spec, tp)
    full, loc = ParamLayout(spec), ParamLayout(ls)
    hq, hk, f = ls.num_heads * ls.head_dim, ls.num_kv_heads * ls.head_dim, ls.intermediate_size
    for name, e in full.entries.items():
        le = loc.entries[name]
        leaf = name.split(".", 1)[-1]
        C = e.shape[1] if len(e.shape) == 2 else 1  # columns of the full tensor
        if leaf in ("wqkv", "bqkv"):
            q0, k0, v0 = 0, spec.q_dim, spec.q_dim + spec.kv_dim
            for r in range(tp):
                for g0, n, l0 in ((q0 + r * hq, hq, 0), (k0 + r * hk, hk, hq), (v0 + r * hk, hk, hq + hk)):
                    yield e.offset + g0 * C, 1, n * C, 0, le.offset + l0 * C, 0, r
        elif leaf == "w_gate_up":
            F = spec.intermediate_size
            for r in range(tp):
                for g0, l0 in ((r * f, 0), (F + r * f, f)):
                    yield e.offset + g0 * C, 1, f * C, 0, le.offset + l0 * C, 0, r
        elif leaf in ("wo", "w_down"):
            w = hq if leaf == "wo" else f  # columns every rank keeps
            for r in range(tp):
                yield e.offset + r * w, e.shape[0], w, C, le.offset, w, r
        else:
            yield e.offset, 1, e.numel, 0, le.offset, 0, -1


def tp_push_plan(spec, tp: int, lo: int, hi: int, n_engines: int = 1, tile_elems: int = 1 << 16, src_shift: int = 0):
    """Copy tiles (numpy structured array, ``TILE_DTYPE``) that move the source range ``[lo, hi)`` of the FULL flat layout
    into the local layouts of ``n_engines`` x ``tp`` engine ranks (destination index ``e * tp + r``).  ``src_shift`` is
    added to every source offset (a learner that holds only a slice of the parameters pushes from its shard buffer)."""
    import numpy as np

    all_ranks = (1 << tp) - 1
    rep = sum(1 << (e * tp) for e in range(n_engines))  # the same rank of every engine
    out = []

    def emit(src, rows, row_len, ss, dst, ds, mask):
        if rows <= 0 or row_len <= 0:
            return
        if rows == 1:  # contiguous: chop into tiles
            for o in range(0, row_len, tile_elems):
                n = min(tile_elems, row_len - o)
                out.append((src + o + src_shift, dst + o, 0, 0, 1, n, mask, 0))
        else:
            per = max(1, tile_elems // row_len)
            for r0 in range(0, rows, per):
                n = min(per, rows - r0)
                out.append((src + r0 * ss + src_shift, dst + r0 * ds, ss, ds, n, row_len, mask, 0))

    for src, rows, row_len, ss, dst, ds, rank in _tp_pieces(spec, tp):
        mask = (all_ranks if rank < 0 else (1 << rank)) * rep
        if rows == 1:
            a, b = max(src, lo), min(src + row_len, hi)
            emit(a, 1, b - a, 0, dst + (a - src), 0, mask)
            continue
        # 2-D piece: rows wholly inside the range go as one strided block, cut rows at either end as single rows
        end = src + (rows - 1) * ss + row_len
        if end <= lo or src >= hi:
            continue
        first = max(0, -(-(lo - src) // ss)) if lo > src else 0            # first row starting at or after lo
        last = min(rows, (hi - src - row_len) // ss + 1) if hi < end else rows  # rows ending at or before hi
        last = max(last, first)
        if first > 0:  # the row before ``first`` may straddle lo
            rs = src + (first - 1) * ss
            a, b = max(rs, lo), min(rs + row_len, hi)
            emit(a, 1, b - a, 0, dst + (first - 1) * ds + (a - rs), 0, mask)
        emit(src + first * ss, last - first, row_len, ss, dst + first * ds, ds, mask)
        if last < rows:  # the row after the block may straddle hi
            rs = src + last * ss
            a, b = max(rs, lo), min(rs + row_len, hi)
            emit(a, 1, b - a, 0, dst + last * ds + (a - rs), 0, mask)
    return np.array(out, dtype=TILE_DTYPE) if out else np.zeros(0, dtype=TILE_DTYPE)


def apply_plan_reference(plan, src: torch.Tensor, dsts: list[torch.Tensor]) -> None:
    """The copy the push kernel performs, in PyTorch (CPU engines, and the oracle of the kernel's test)."""
    with torch.no_grad():
        for t in plan:
            for d, dst in enumerate(dsts):
                if not (int(t["mask"]) >> d) & 1:
                    continue
                for r in range(int(t["rows"])):
                    so, do, n = int(t["src"]) + r * int(t["src_stride"]), int(t["dst"]) + r * int(t["dst_stride"]), int(t["row_len"])
                    dst[do:do + n].copy_(src[so:so + n].to(dst.dtype))


def push_tp(src: torch.Tensor, dsts: list, plan_dev: torch.Tensor, n_tiles: int) -> None:
    """Run the tensor-parallel push kernel: ``plan_dev`` is the tile table (``tp_push_plan``) as a uint8 CUDA tensor."""
    so = lib.load_ops()
    for d in dsts:
        if isinstance(d, PeerBuffer):
            if d.mapped_for != src.device.index:
                raise ValueError(f"buffer was mapped for GPU {d.mapped_for} but the push runs on GPU {src.device.index}")
        else:
            ensure_peer_access(src.device.index, d.device.index)
    arr = (ctypes.c_void_p * 8)()
    for i, d in enumerate(dsts):
        arr[i] = d.data_ptr()
    fn = so.b200_tp_push
    fn.argtypes, fn.restype = lib._SIGNATURES["b200_tp_push"], _I
    with torch.cuda.device(src.device):
        rc = fn(ptr(src), arr, len(dsts), ptr(plan_dev), n_tiles, int(src.dtype == torch.float32), stream_ptr())
    lib.launch_count += 1
    if rc:
        raise lib.KernelError(f"b200_tp_push failed with code {rc}")


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
            e.engine.reset_prefix_cache()  # K/V kept for later requests belong to the old weights
    finally:
        for e in engines:
            e.lock.release()
    return time.perf_counter() - t0
