"""Symmetric-memory state of the learner group and the fused optimizer-step collectives.

The bf16 working parameters and the fp32 gradient accumulator of every rank are allocated in
symmetric memory (``torch.distributed._symmetric_memory`` does the allocation, the handle
exchange between the rank processes and the optional NVLS multicast binding - that is plumbing).
Everything that moves data is done by this package's own kernels
(``open_instruct_b200/ops/csrc/zero_comm.cu``), which dereference the peers' pointers directly:

* ``reduce_scatter_grad``  barrier, then each owner sums its slice out of all peers' gradient
  buffers, accumulating the squared norm in the same pass; norms are exchanged through the
  signal pads.  (What DeepSpeed does with bucketed NCCL reduce-scatter + a separate norm pass.)
* ``adamw_allgather``      AdamW on the owner's fp32 shard with the bf16 result stored into every
  peer's working copy from inside the optimizer kernel.  (DeepSpeed: optimizer step, bf16 copy,
  then NCCL all-gather.)
* ``finish_step``          barrier: all stores have landed.
* ``reduce_ready_range``   the overlapped form of the reduce-scatter: while the LAST micro-batch's backward is still
  running, every range of the gradient buffer that has received its final contribution (one decoder layer at a time)
  is reduced by its owner on a side stream - an event from the compute stream, a device barrier on the side stream's own
  flag row (all ranks have finished that range), then the same reduce kernel on a small grid that shares the SMs with
  the backward GEMMs.  ``reduce_scatter_grad`` afterwards only reduces what is left (embedding, norm weights).  This
  is the schedule DeepSpeed's ``overlap_comm`` gives the reference (``open_instruct/utils.py:1431-1460``), with the
  gradients still crossing NVLink once per optimizer step instead of once per micro-batch.

``use_multimem=True`` switches the two data kernels to ``multimem.ld_reduce`` / ``multimem.st`` through
the NVSwitch when the allocation has a multicast address.  Waits on peers are bounded
(``peer_timeout_ms``): a rank whose peer never arrives gets ``ST_TIMEOUT_PEER`` in the status word and
an exception at the end of that optimizer step (``Learner.optimizer_step`` reads the status word) instead of a hung GPU.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import lib
from ..ops.lib import ptr, status_word, stream_ptr

_P, _I, _L, _F, _U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint
_PP = ctypes.POINTER(ctypes.c_void_p)

lib._SIGNATURES.update({
    "b200_symm_barrier": [_PP, _I, _I, _U, _I, _P, _P],
    "b200_symm_allreduce_scalar": [_PP, _I, _I, _U, _P, _P, _I, _P, _P],
    "b200_symm_barrier_side": [_PP, _I, _I, _U, _I, _P, _P],
    "b200_zero_reduce_scatter": [_PP, _P, _I, _I, _L, _L, _P, _P, _I, _P],
    "b200_zero_reduce_range": [_PP, _P, _I, _L, _L, _P, _P, _I, _I, _P],
    "b200_symm_allreduce_vec": [_PP, _PP, _I, _I, _U, _P, _P, _I, _I, _P, _P],
    "b200_zero_adamw_allgather": [_P, _P, _P, _P, _PP, _P, _I, _L, _L, _P, _F, _F, _F, _F, _F, _I, _I, _P],
})


def unreduced_ranges(lo: int, hi: int, done: list[tuple[int, int]]) -> list[tuple[int, int]]:
    """The parts of ``[lo, hi)`` that none of the (possibly overlapping, unordered) ranges in ``done`` covers."""
    out, pos = [], lo
    for a, b in sorted(done):
        if a > pos:
            out.append((pos, min(a, hi)))
        pos = max(pos, b)
        if pos >= hi:
            break
    if pos < hi:
        out.append((pos, hi))
    return [(a, b) for a, b in out if a < b]


_METRICS_STATE = None  # the SymmetricState whose exchange buffer serves metric reductions over the default group


def metrics_state(group=None):
    """The symmetric state to reduce a metric vector over ``group`` with, if one exists for exactly that group."""
    st = _METRICS_STATE
    if st is None:
        return None
    want = group if group is not None else dist.group.WORLD
    return st if st.group is want else None


def _ptr_array(ptrs) -> ctypes.Array:
    arr = (ctypes.c_void_p * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = int(p)
    return arr


class SymmetricState:
    """Symmetric ``params`` (bf16) and ``grads`` (fp32) buffers of ``n`` elements + their peer maps."""

    def __init__(self, n: int, device, group=None, use_multimem: bool | None = None, peer_timeout_ms: int = 20000):
        import torch.distributed._symmetric_memory as symm_mem

        if not dist.is_initialized():
            raise RuntimeError("SymmetricState needs an initialised process group")
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("one NVSwitch domain: at most 8 ranks")
        self.device = torch.device(device)
        self.n = n
        self.peer_timeout_ms = peer_timeout_ms
        self.params = symm_mem.empty(n, dtype=torch.bfloat16, device=self.device)
        self.grads = symm_mem.empty(n, dtype=torch.float32, device=self.device)
        self.params.zero_()
        self.grads.zero_()
        self._hp = symm_mem.rendezvous(self.params, self.group)
        self._hg = symm_mem.rendezvous(self.grads, self.group)
        self._param_ptrs = _ptr_array(self._hp.buffer_ptrs)
        self._grad_ptrs = _ptr_array(self._hg.buffer_ptrs)
        self._pads = _ptr_array(self._hg.signal_pad_ptrs)
        self._mc_params = int(self._hp.multicast_ptr or 0)
        self._mc_grads = int(self._hg.multicast_ptr or 0)
        if use_multimem is None:
            use_multimem = os.environ.get("B200_MULTIMEM", "0") == "1"
        self.use_multimem = bool(use_multimem and self._mc_params and self._mc_grads)
        self._barrier_epoch = 0
        self._side_epoch = 0
        self._scalar_epoch = 0
        self._local_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        # overlapped exchange: a high-priority side stream, the ranges of MY slice already reduced in this step, and the
        # number of CTAs the side-stream reduce may take from the backward pass
        self.side_stream = torch.cuda.Stream(self.device, priority=-1)
        self._reduced: list[tuple[int, int]] = []
        self._sq_zeroed = False
        self.overlap_ctas = int(os.environ.get("B200_OVERLAP_CTAS", "48"))
        lib.load_ops()
        for name, sig in lib._SIGNATURES.items():
            fn = getattr(lib.load_ops(), name, None)
            if fn is not None:
                fn.argtypes = sig
                fn.restype = ctypes.c_int
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every rank has mapped every peer before any kernel touches them
        self.shard = n // self.world
        # exchange buffer of the small-vector all-reduce (metric vectors of a logging step)
        self._vec_epoch = 0
        self.vec_buf = symm_mem.empty(2 * 8 * 512, dtype=torch.float32, device=self.device)
        self.vec_buf.zero_()
        self._hv = symm_mem.rendezvous(self.vec_buf, self.group)
        self._vec_ptrs = _ptr_array(self._hv.buffer_ptrs)
        self._vec_pads = _ptr_array(self._hv.signal_pad_ptrs)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        global _METRICS_STATE
        _METRICS_STATE = self

    def allreduce_vector_(self, vec: torch.Tensor) -> torch.Tensor:
        """In-place sum over the ranks of a small fp32 vector (at most 512 entries) in ONE kernel over symmetric memory:
        no library collective on the logging path.  The parity of the epoch alternates the exchange slots, so a rank that
        races ahead into the next reduction cannot overwrite values a slower rank is still adding."""
        if vec.dtype != torch.float32 or not vec.is_cuda or vec.numel() > 512 or not vec.is_contiguous():
            raise ValueError("allreduce_vector_ takes a contiguous CUDA fp32 vector of at most 512 entries")
        self._vec_epoch += 1
        lib.call("b200_symm_allreduce_vec", self._vec_ptrs, self._vec_pads, self.rank, self.world, self._vec_epoch, ptr(vec), ptr(vec),
                 vec.numel(), self.peer_timeout_ms, ptr(status_word(self.device)), stream_ptr())
        return vec

    # ------------------------------------------------------------------ primitives
    def barrier(self) -> None:
        """Device-side barrier on the current stream (no host synchronisation)."""
        self._barrier_epoch += 1
        lib.call("b200_symm_barrier", self._pads, self.rank, self.world, self._barrier_epoch, self.peer_timeout_ms,
                 ptr(status_word(self.device)), stream_ptr())

    def allreduce_scalar(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        self._scalar_epoch += 1
        lib.call("b200_symm_allreduce_scalar", self._pads, self.rank, self.world, self._scalar_epoch, ptr(src), ptr(dst),
                 self.peer_timeout_ms, ptr(status_word(self.device)), stream_ptr())

    # ------------------------------------------------------------------ optimizer-step collectives
    def _reduce_range(self, a: int, b: int, out_shard: torch.Tensor, ctas: int) -> None:
        """Sum ``grads[a:b]`` (global element offsets inside my slice) over the ranks into ``out_shard``."""
        lo = self.rank * self.shard
        lib.call("b200_zero_reduce_range", self._grad_ptrs, self._mc_grads or None, self.world, a, b - a,
                 out_shard[a - lo:].data_ptr(), ptr(self._local_sq), int(self.use_multimem), ctas, stream_ptr())

    def reduce_ready_range(self, lo: int, hi: int, out_shard: torch.Tensor) -> None:
        """Every rank calls this, in the same order, once ``grads[lo:hi]`` has received its last contribution of the
        step on the current stream.  The owner of each part of the range reduces it on the side stream, beside whatever
        the current stream runs next."""
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        with torch.cuda.stream(self.side_stream):
            self.side_stream.wait_event(ev)
            if not self._sq_zeroed:
                self._local_sq.zero_()
                self._sq_zeroed = True
            self._side_epoch += 1
            lib.call("b200_symm_barrier_side", self._pads, self.rank, self.world, self._side_epoch, self.peer_timeout_ms,
                     ptr(status_word(self.device)), stream_ptr())
            my_lo = self.rank * self.shard
            a, b = max(lo, my_lo), min(hi, my_lo + self.shard)
            a, b = (a + 3) // 4 * 4, b // 4 * 4
            if a < b:
                self._reduce_range(a, b, out_shard, self.overlap_ctas)
                self._reduced.append((a, b))

    def reduce_scatter_grad(self, out_shard: torch.Tensor, norm_sq: torch.Tensor) -> torch.Tensor:
        """``out_shard`` = sum over ranks of my slice of ``grads``; ``norm_sq`` = global |sum grad|^2.  Ranges that
        ``reduce_ready_range`` already reduced in this step are skipped."""
        main = torch.cuda.current_stream(self.device)
        if self._reduced or self._sq_zeroed:
            main.wait_stream(self.side_stream)
        if not self._sq_zeroed:
            self._local_sq.zero_()
        self.barrier()  # every rank's backward has finished writing its gradient buffer
        my_lo = self.rank * self.shard
        for a, b in unreduced_ranges(my_lo, my_lo + self.shard, self._reduced):
            self._reduce_range(a, b, out_shard, 0)
        self._reduced, self._sq_zeroed = [], False
        # also the point after which every rank has finished READING the peers' gradients
        self.allreduce_scalar(self._local_sq, norm_sq)
        return out_shard

    def adamw_allgather(self, master, m, v, grad, global_offset: int, *, gscale, lr, beta1, beta2, eps, wd, step) -> None:
        lib.call("b200_zero_adamw_allgather", ptr(master), ptr(m), ptr(v), ptr(grad), self._param_ptrs,
                 self._mc_params or None, self.world, global_offset, master.numel(), ptr(gscale), lr, beta1, beta2, eps,
                 wd, step, int(self.use_multimem), stream_ptr())

    def finish_step(self) -> None:
        self.barrier()
