"""ctypes binding to ``libb200ops.so`` (the sm_100a kernels) and ``libb200host.so``.

The kernels export a plain C ABI taking raw device pointers and a CUDA stream, so the same
library serves PyTorch tensors here and any other caller.  On a machine with a GPU the
library MUST load: there is no silent PyTorch fallback for the fused path; a missing library
raises.  On a CPU-only machine ``available()`` is False and the ``ref`` ops are used.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_OPS_PATH = _HERE / "libb200ops.so"
_HOST_PATH = _HERE / "libb200host.so"
_lock = threading.Lock()
_ops = None
_host = None

P, I, L, F = c_void_p, c_int, c_longlong, c_float

# name -> argtypes; every function returns int (0 = ok, else CUDA / driver error code)
_SIGNATURES = {
    "b200_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, P, P, I],
    "b200_gemm2_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, P, P, I],
    "b200_gemm_bf16_skinny": [P, P, P, I, I, I, L, L, L, P, P, I],
    "b200_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "b200_rope_table": [P, P, P, I, I, P],
    "b200_rope_apply": [P, P, I, I, I, I, I, P],
    "b200_rmsnorm_fwd_acc32": [P, P, P, P, P, P, I, I, F, P],
    "b200_gemm_bf16_splitk": [P, P, P, I, I, I, L, L, L, I, P, P],
    "b200_gemm_decode": [P, P, P, I, I, I, L, L, L, L, I, I, I, P, P],
    "b200_rmsnorm_fwd_parts": [P, I, L, P, P, P, P, I, I, F, P],
    "b200_rmsnorm_bwd_ctas": [I],
    "b200_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, P],
    "b200_rope": [P, P, P, I, I, I, I, I, P],
    "b200_swiglu_fwd": [P, P, L, I, P],
    "b200_swiglu_bwd": [P, P, P, L, I, P],
    "b200_embedding_fwd": [P, P, P, I, I, I, P],
    "b200_embedding_bwd": [P, P, P, I, I, I, P],
    "b200_sumsq_scratch_floats": [],
    "b200_sumsq": [P, L, P, P, I, P],
    "b200_adamw": [P, P, P, P, P, L, P, F, F, F, F, F, I, I, P],
    "b200_cast_f32_bf16": [P, P, L, F, P],
    "b200_accum_bf16_f32": [P, P, L, P],
    "b200_logprob_fwd": [P, P, P, P, P, I, I, L, F, P],
    "b200_logprob_bwd": [P, P, P, P, I, I, L, F, P],
    "b200_logprob_fwd_vp": [P, P, P, P, P, I, I, L, F, L, P],
    "b200_logprob_bwd_vp": [P, P, P, P, I, I, L, F, L, P],
    "b200_kv_write": [P, P, P, P, I, I, I, I, I, P],
    "b200_paged_decode": [P, P, P, P, I, P, I, I, I, I, F, I, P, P, P, P],
    "b200_paged_decode_variant": [I],
    "b200_rope_kv_decode": [P, P, P, P, P, I, I, I, I, P],
    "b200_sample": [P, L, I, I, P, P, P, P, P, P, P],
    "b200_attn_fwd": [P, P, P, P, P, I, I, I, I, I, I, F, P],
    "b200_attn_bwd": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, P],
}


class KernelError(RuntimeError):
    """A kernel launch failed or one of its bounded waits ran out."""


def ops_library_path() -> Path:
    return _OPS_PATH


def load_ops():
    """Load (building first if the shared object is missing and nvcc exists)."""
    global _ops
    with _lock:
        if _ops is not None:
            return _ops
        if not _OPS_PATH.exists():
            from . import build

            build.build_ops(verbose=False)
        lib = ctypes.CDLL(str(_OPS_PATH))
        for name, argtypes in _SIGNATURES.items():
            if hasattr(lib, name):
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = c_int
        _ops = lib
        return lib


def load_host():
    global _host
    with _lock:
        if _host is not None:
            return _host
        if not _HOST_PATH.exists():
            from . import build

            build.build_host(verbose=False)
        _host = ctypes.CDLL(str(_HOST_PATH))
        return _host


def available() -> bool:
    """True when the fused sm_100a path can run in this process."""
    if not torch.cuda.is_available():
        return False
    major, _ = torch.cuda.get_device_capability()
    if major != 10:
        return False
    load_ops()  # raises when the library is missing on a GPU machine: fail loudly
    return True


def ptr(t):
    """Device pointer of a tensor (``None`` -> NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_status = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 status word the tcgen05 kernels write when a bounded wait runs out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = t
    return t


_status_host = {}


def check_status(sync: bool = True) -> None:
    """Raise ``KernelError`` when any kernel recorded a timed-out wait.

    ``sync=True`` reads the status word now (synchronises the device).  ``sync=False`` never blocks: it looks at the copy
    of the word that the PREVIOUS non-blocking call queued (raising if that copy has arrived and is non-zero) and queues
    a fresh copy into pinned host memory behind the work submitted so far, so a failure surfaces one call later."""
    for key, t in _status.items():
        if sync:
            code = int(t.item())
        else:
            slot = _status_host.get(key)
            if slot is None:
                slot = _status_host[key] = [torch.zeros(1, dtype=torch.int32, pin_memory=True), torch.cuda.Event(), False]
            host, ev, pending = slot
            code = 0
            if pending and ev.query():
                code = int(host[0])
            if not pending or ev.query():
                with torch.cuda.device(t.device):
                    host.copy_(t, non_blocking=True)
                    ev.record(torch.cuda.current_stream(t.device))
                slot[2] = True
        if code:
            t.zero_()
            raise KernelError(f"kernel on cuda:{key} gave up a bounded wait (status {code})")


# kernels launched per library call (for launch accounting in benchmarks)
_KERNELS_PER_CALL = {"b200_attn_bwd": 3, "b200_rmsnorm_bwd": 2, "b200_sumsq": 2, "b200_allgather_copy": 0}
launch_count = 0


def call(name: str, *args) -> None:
    global launch_count
    lib = load_ops()
    launch_count += _KERNELS_PER_CALL.get(name, 1)
    fn = getattr(lib, name)
    if fn.argtypes is None and name in _SIGNATURES:  # registered by a module imported after the library was loaded
        fn.argtypes, fn.restype = _SIGNATURES[name], c_int
    rc = fn(*args)
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}")
