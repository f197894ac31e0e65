"""Symmetric-memory transport of the parameter-sharded learner: pull-gather of parameter slices and the per-layer
gradient reduction, both by this package's kernels over peer pointers (``ops/csrc/zero_comm.cu``).

The bf16 parameter slices of a rank and its two layer-sized fp32 gradient workspaces live in symmetric memory.  A gather
reads the same slice range out of every peer's buffer (no handshake: parameters are constant between optimizer steps,
and ``Zero3State`` fences the step with ``barrier``).  A reduction is ``barrier`` (every rank's backward of that layer
has been written) followed by a kernel in which the owner sums its slice out of every rank's workspace into its gradient
shard.  Replaces what the reference gets from DeepSpeed's bucketed NCCL all-gather / reduce-scatter
(``configs/ds_configs/stage3_no_offloading_accelerate.conf``: ``overlap_comm``, ``stage3_prefetch_bucket_size``).
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import lib
from ..ops.lib import ptr, status_word, stream_ptr
from .symm import _ptr_array

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_PP = ctypes.POINTER(ctypes.c_void_p)

lib._SIGNATURES.update({
    "b200_allgather_pull": [_PP, _I, _L, _L, _P, _I, _P],
    "b200_reduce_scatter_add": [_PP, _P, _I, _L, _L, _P, _I, _P],
    "b200_allgather_copy": [_PP, _I, _L, _L, _I, _P, _P],
})


class PeerComm:
    def __init__(self, n_shards: int, ws: int, device, group=None, peer_timeout_ms: int = 20000):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("one NVSwitch domain: at most 8 ranks")
        self.device = torch.device(device)
        self.peer_timeout_ms = peer_timeout_ms
        self.shards = symm_mem.empty(n_shards, dtype=torch.bfloat16, device=self.device)
        self.grad_ws = [symm_mem.empty(ws, dtype=torch.float32, device=self.device) for _ in range(2)]
        self.shards.zero_()
        hs = symm_mem.rendezvous(self.shards, self.group)
        self._shard_ptrs = _ptr_array(hs.buffer_ptrs)
        self._pads = _ptr_array(hs.signal_pad_ptrs)
        self._ws_ptrs, self._ws_mc = [], []
        # B200_MULTIMEM=1: the reduction reads through the workspaces' multicast address (the NVSwitch adds the ranks'
        # values); off by default, like the optimizer-step kernels' multimem variants
        want_mc = os.environ.get("B200_MULTIMEM", "0") == "1"
        for w in self.grad_ws:
            w.zero_()
            hw = symm_mem.rendezvous(w, self.group)
            self._ws_ptrs.append(_ptr_array(hw.buffer_ptrs))
            self._ws_mc.append(int(hw.multicast_ptr or 0) if want_mc else 0)
        self.use_multimem = all(self._ws_mc)
        self._handles = hs
        self._epoch = 0
        # CTAs of the two transport kernels: they run beside the layer's GEMMs, so they get a slice of the SMs only
        # the gather goes through the copy engines by default ("ce": no SM taken from the GEMMs); "sm" = the pull kernel
        self.gather_mode = os.environ.get("B200_Z3_GATHER", "ce")
        self.gather_ctas = int(os.environ.get("B200_Z3_GATHER_CTAS", "64"))
        self.reduce_ctas = int(os.environ.get("B200_Z3_REDUCE_CTAS", "64"))
        lib.load_ops()
        for name in ("b200_symm_barrier", "b200_allgather_pull", "b200_reduce_scatter_add", "b200_allgather_copy"):
            fn = getattr(lib.load_ops(), name)
            fn.argtypes = lib._SIGNATURES[name]
            fn.restype = ctypes.c_int
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def barrier(self) -> None:
        """Device-side barrier on the current stream; bounded (a missing peer sets the status word)."""
        self._epoch += 1
        lib.call("b200_symm_barrier", self._pads, self.rank, self.world, self._epoch, self.peer_timeout_ms,
                 ptr(status_word(self.device)), stream_ptr())

    def all_gather(self, out: torch.Tensor, soff: int, n: int) -> None:
        if self.gather_mode == "ce":
            lib.call("b200_allgather_copy", self._shard_ptrs, self.world, soff, n, 2, ptr(out), stream_ptr())
        else:
            lib.call("b200_allgather_pull", self._shard_ptrs, self.world, soff, n, ptr(out), self.gather_ctas, stream_ptr())

    def reduce_scatter_add(self, slot: int, n: int, acc: torch.Tensor) -> None:
        self.barrier()  # every rank has finished writing this workspace
        lib.call("b200_reduce_scatter_add", self._ws_ptrs[slot], self._ws_mc[slot] if self.use_multimem else None, self.world,
                 self.rank * n, n, ptr(acc), self.reduce_ctas, stream_ptr())
        self.barrier()  # every rank has finished reading it: whoever waits on this stream may overwrite its copy
