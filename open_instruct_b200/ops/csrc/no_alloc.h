// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference framework, which owns no native code.
// It exists for callers that cannot allocate device memory at the moment they need the op:
// code running inside a memory pool it must not disturb, a host that hands the library fixed
// buffers only, or a runtime whose allocator may not be re-entered from where the call is made.
// Everything else in this library takes its scratch space from the caller.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// RMSNorm backward with built-in scratch.  Same arguments and results as b200_rmsnorm_bwd minus
// the `dw_partial` scratch pointer:
//   h, w, dy, dres (optional), dx : bf16;  rstd : fp32 [T];  dw_out (optional): fp32 [D], accumulated into.
//
// * Scratch: a fixed 296 x 8192 float array (9.25 MiB) inside the library image.  Every GPU
//   whose context loads the library holds it until the process exits.
// * Limit: D <= 8192 (b200_rmsnorm_bwd_noalloc_max_d()); larger D returns -3 with a message on
//   stderr and launches nothing.  D must be a multiple of 8.
// * The call itself performs no cudaMalloc / cudaFree and uses no allocating library routine.
// * The first call on each device resolves the array's device address (with that device
//   current) and sets the kernel's shared-memory attribute; make that first call outside any
//   stream capture.  Later calls only launch.
// * All calls on a device share the one array.  Nothing in it needs clearing between calls
//   (each launch overwrites the rows it later reads), but two calls whose kernels overlap on
//   the GPU - different streams without an ordering between them - race on it.  Keep calls on
//   one stream or order them with events.
// Returns 0, or a negative argument error, or a CUDA error code.
int b200_rmsnorm_bwd_noalloc(const void* h, const void* w, const float* rstd, const void* dy, const void* dres,
                             void* dx, float* dw_out, int T, int D, void* stream);

// Largest D the entry point above accepts.
int b200_rmsnorm_bwd_noalloc_max_d(void);

#ifdef __cplusplus
}
#endif
