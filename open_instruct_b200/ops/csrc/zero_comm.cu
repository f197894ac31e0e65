// Optimizer-step collectives fused with their compute, over NVLink peer memory.
//
// Every rank holds its fp32 gradient buffer and its bf16 working parameters in symmetric
// memory (same layout on every GPU, every peer's copy mapped locally).  Per optimizer step:
//
//   symm_barrier            all ranks' backward kernels have finished (flag exchange, bounded)
//   zero_reduce_scatter     owner reads its slice from EVERY peer's gradient buffer with P2P
//                           loads (or one multimem.ld_reduce through the switch), sums in fp32,
//                           writes the reduced shard and accumulates its squared norm
//   symm_allreduce_scalar   squared norms exchanged through the signal pads (deterministic order)
//   zero_adamw_allgather    AdamW on the fp32 shard; the refreshed bf16 values are stored straight
//                           into every peer's working copy (P2P stores, or one multimem.st)
//   symm_barrier            all stores have landed before anyone starts the next forward
//
// No TMA is used here: all remote traffic is ordinary ld/st (or multimem) from this GPU's SMs.
// Every wait is bounded and reports through the status word instead of hanging.
#include "common.cuh"
#include "peer.cuh"

namespace b200 {

// One thread per peer: publish my arrival in the peer's pad, then wait for the peer's in mine.
// `slot`: first pad word of the flag row used (PAD_BARRIER, or PAD_BARRIER_SIDE for barriers issued on a second stream:
// the wait is "flag >= epoch", so two streams must not share a row).
__global__ void symm_barrier_kernel(PeerPtrs pads, int rank, int world, uint32_t epoch, long long limit_cycles,
                                    int* __restrict__ status, int slot) {
  const int peer = threadIdx.x;
  if (peer >= world) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<uint32_t*>(pads.p[peer]) + slot + rank, epoch);
  if (!wait_epoch(reinterpret_cast<const uint32_t*>(pads.p[rank]) + slot + peer, epoch, limit_cycles))
    atomicCAS(status, 0, ST_TIMEOUT_PEER);
}

// out[0] = sum over ranks of in[0], summed in rank order on every rank (bitwise identical everywhere).
__global__ void symm_allreduce_scalar_kernel(PeerPtrs pads, int rank, int world, uint32_t epoch,
                                             const float* __restrict__ in, float* __restrict__ out,
                                             long long limit_cycles, int* __restrict__ status) {
  __shared__ int failed;
  const int peer = threadIdx.x;
  const int par = epoch & 1;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (peer < world) {
    uint32_t* pad = reinterpret_cast<uint32_t*>(pads.p[peer]);
    reinterpret_cast<volatile float*>(pad)[PAD_SCALAR_VAL + par * 8 + rank] = in[0];
    __threadfence_system();
    st_release_sys(pad + PAD_SCALAR_FLAG + rank, epoch);
    if (!wait_epoch(reinterpret_cast<const uint32_t*>(pads.p[rank]) + PAD_SCALAR_FLAG + peer, epoch, limit_cycles)) {
      atomicCAS(status, 0, ST_TIMEOUT_PEER);
      failed = 1;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    if (!failed) {
      const volatile float* mine = reinterpret_cast<const volatile float*>(pads.p[rank]) + PAD_SCALAR_VAL + par * 8;
      for (int r = 0; r < world; ++r) s += mine[r];
    } else {
      s = in[0];
    }
    out[0] = s;
  }
}

// out[i] = sum over ranks of in[i], i < n <= SYMM_VEC_MAX: the one small reduction a logging step needs (metric vectors).
// `bufs.p[r]` is rank r's symmetric exchange buffer of 2 (parity) x MAX_PEERS x SYMM_VEC_MAX floats: every rank stores its
// vector into its own slot of EVERY peer's buffer, raises its flag there, waits (bounded) for everyone's flag in its own pad
// and adds the slots of its own buffer in rank order, so the result is bitwise the same on every rank.  One CTA.
constexpr int SYMM_VEC_MAX = 512;
__global__ void __launch_bounds__(512)
symm_allreduce_vec_kernel(PeerPtrs bufs, PeerPtrs pads, int rank, int world, uint32_t epoch, const float* __restrict__ in,
                          float* __restrict__ out, int n, long long limit_cycles, int* __restrict__ status) {
  __shared__ int failed;
  const int par = epoch & 1;
  if (threadIdx.x == 0) failed = 0;
  for (int r = 0; r < world; ++r) {
    float* slot = reinterpret_cast<float*>(bufs.p[r]) + (static_cast<long long>(par) * MAX_PEERS + rank) * SYMM_VEC_MAX;
    for (int i = threadIdx.x; i < n; i += blockDim.x) reinterpret_cast<volatile float*>(slot)[i] = in[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) {
    st_release_sys(reinterpret_cast<uint32_t*>(pads.p[threadIdx.x]) + PAD_VEC_FLAG + rank, epoch);
    if (!wait_epoch(reinterpret_cast<const uint32_t*>(pads.p[rank]) + PAD_VEC_FLAG + threadIdx.x, epoch, limit_cycles)) {
      atomicCAS(status, 0, ST_TIMEOUT_PEER);
      failed = 1;
    }
  }
  __syncthreads();
  const volatile float* mine = reinterpret_cast<const volatile float*>(bufs.p[rank]) + static_cast<long long>(par) * MAX_PEERS * SYMM_VEC_MAX;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float s = 0.f;
    if (!failed) {
      for (int r = 0; r < world; ++r) s += mine[r * SYMM_VEC_MAX + i];
    } else {
      s = in[i];  // a peer never arrived: the local values stand, the status word tells the host
    }
    out[i] = s;
  }
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b128(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

// out[i] = sum_r grads_r[lo + i],  i in [0, n);  sumsq += sum out[i]^2.   n % 4 == 0.
// P2P variant: a peer load takes a few microseconds over NVLink, so the achieved rate is (bytes in flight) / latency.
// Every thread therefore issues the loads of ALL ranks for U vectors (up to 16 independent 16-byte loads) before the
// first add; the adds then run in fixed rank order, which keeps the sum bitwise identical from run to run.
// MULTIMEM variant: one `multimem.ld_reduce` returns the sum over all ranks (the NVSwitch adds), so the owner's ingress
// carries n floats instead of world * n.
// U: vectors per thread per round; the launcher picks it so that U * world is about 16 loads in flight per thread
// whatever the number of ranks (with two ranks and U = 2 a small grid reached only a fifth of the link rate).
template <bool MULTIMEM, int U, int W>
__global__ void __launch_bounds__(256)
zero_reduce_scatter_kernel(PeerPtrs grads, const float* __restrict__ mc_grads, int world, long long lo,
                           long long n, float* __restrict__ out, float* __restrict__ sumsq) {
  __shared__ float red[8];
  float ss = 0.f;
  const long long nv = n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nv; i0 += stride * U) {
    if (MULTIMEM) {
      float4 a[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nv) a[u] = multimem_ld_reduce_f32x4(mc_grads + lo + i * 4);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nv) {
          reinterpret_cast<float4*>(out)[i] = a[u];
          ss += a[u].x * a[u].x + a[u].y * a[u].y + a[u].z * a[u].z + a[u].w * a[u].w;
        }
      }
    } else {
      uint4 x[U][W];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
#pragma unroll
        for (int r = 0; r < W; ++r)
          if (r < world && i < nv)
            x[u][r] = ld_volatile_u4(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo) + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nv) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int r = 0; r < W; ++r)
            if (r < world) {
              acc.x += __uint_as_float(x[u][r].x); acc.y += __uint_as_float(x[u][r].y);
              acc.z += __uint_as_float(x[u][r].z); acc.w += __uint_as_float(x[u][r].w);
            }
          reinterpret_cast<float4*>(out)[i] = acc;
          ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) atomicAdd(sumsq, v);
  }
}

// AdamW on n (multiple of 8) fp32 elements; bf16 result stored at element offset `goff` of every
// peer's parameter buffer.
template <bool MULTIMEM>
__global__ void __launch_bounds__(256)
zero_adamw_allgather_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                            const float* __restrict__ grad, PeerPtrs params, void* mc_params, int world, long long goff,
                            long long n, const float* __restrict__ gscale, float lr, float beta1, float beta2,
                            float eps, float wd, float bc1, float bc2) {
  const float gs = gscale ? gscale[0] : 1.f;
  const long long nv = n / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float p[8], mm[8], vv[8], g[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 a = reinterpret_cast<const float4*>(master)[i * 2 + h];
      const float4 b = reinterpret_cast<const float4*>(m)[i * 2 + h];
      const float4 c = reinterpret_cast<const float4*>(v)[i * 2 + h];
      const float4 d = reinterpret_cast<const float4*>(grad)[i * 2 + h];
      p[4 * h] = a.x; p[4 * h + 1] = a.y; p[4 * h + 2] = a.z; p[4 * h + 3] = a.w;
      mm[4 * h] = b.x; mm[4 * h + 1] = b.y; mm[4 * h + 2] = b.z; mm[4 * h + 3] = b.w;
      vv[4 * h] = c.x; vv[4 * h + 1] = c.y; vv[4 * h + 2] = c.z; vv[4 * h + 3] = c.w;
      g[4 * h] = d.x; g[4 * h + 1] = d.y; g[4 * h + 2] = d.z; g[4 * h + 3] = d.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gs;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      p[j] *= (1.f - lr * wd);
      p[j] -= lr * (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(master)[i * 2 + h] = make_float4(p[4 * h], p[4 * h + 1], p[4 * h + 2], p[4 * h + 3]);
      reinterpret_cast<float4*>(m)[i * 2 + h] = make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
      reinterpret_cast<float4*>(v)[i * 2 + h] = make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
    }
    uint4 pk;
    pk.x = pack_bf16x2(p[0], p[1]);
    pk.y = pack_bf16x2(p[2], p[3]);
    pk.z = pack_bf16x2(p[4], p[5]);
    pk.w = pack_bf16x2(p[6], p[7]);
    if (MULTIMEM) {
      multimem_st_b128(reinterpret_cast<__nv_bfloat16*>(mc_params) + goff + i * 8, pk);
    } else {
#pragma unroll 1
      for (int r = 0; r < world; ++r)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + goff + i * 8) = pk;
    }
  }
}


}  // namespace b200

using namespace b200;

// `limit_ms`: how long a rank waits for its peers before it records ST_TIMEOUT_PEER and returns.
extern "C" int b200_symm_barrier(const void* const* pad_ptrs, int rank, int world, unsigned epoch, int limit_ms,
                                 int* status, void* stream) {
  if (world > MAX_PEERS) return -1;
  const long long cycles = static_cast<long long>(limit_ms) * 1900000LL;
  symm_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_ptrs(pad_ptrs, world), rank, world,
                                                                         epoch, cycles, status, PAD_BARRIER);
  return static_cast<int>(cudaGetLastError());
}

// The same barrier on its own flag row, for a second stream that runs beside the one using `b200_symm_barrier`
// (the gradient exchange that overlaps the backward pass).  Epochs of the two rows count independently.
extern "C" int b200_symm_barrier_side(const void* const* pad_ptrs, int rank, int world, unsigned epoch, int limit_ms,
                                      int* status, void* stream) {
  if (world > MAX_PEERS) return -1;
  const long long cycles = static_cast<long long>(limit_ms) * 1900000LL;
  symm_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_ptrs(pad_ptrs, world), rank, world,
                                                                         epoch, cycles, status, PAD_BARRIER_SIDE);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_symm_allreduce_scalar(const void* const* pad_ptrs, int rank, int world, unsigned epoch,
                                          const float* in, float* out, int limit_ms, int* status, void* stream) {
  if (world > MAX_PEERS) return -1;
  const long long cycles = static_cast<long long>(limit_ms) * 1900000LL;
  symm_allreduce_scalar_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_ptrs(pad_ptrs, world), rank, world, epoch, in, out, cycles, status);
  return static_cast<int>(cudaGetLastError());
}

// Floats of the exchange buffer `b200_symm_allreduce_vec` needs per rank (allocate it in symmetric memory, zeroed).
extern "C" int b200_symm_vec_buffer_floats() { return 2 * MAX_PEERS * SYMM_VEC_MAX; }

extern "C" int b200_symm_allreduce_vec(const void* const* buf_ptrs, const void* const* pad_ptrs, int rank, int world, unsigned epoch,
                                       const float* in, float* out, int n, int limit_ms, int* status, void* stream) {
  if (world > MAX_PEERS || n < 0 || n > SYMM_VEC_MAX) return -1;
  if (n == 0) return 0;
  const long long cycles = static_cast<long long>(limit_ms) * 1900000LL;
  symm_allreduce_vec_kernel<<<1, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_ptrs(buf_ptrs, world), make_ptrs(pad_ptrs, world), rank,
                                                                               world, epoch, in, out, n, cycles, status);
  return static_cast<int>(cudaGetLastError());
}

// Parameter sharding (gather on use).  out[r * n + i] = shard_r[soff + i] for every rank r: each GPU PULLS the peers'
// slices with 16-byte loads (its own slice is an ordinary local copy).  Parameters only change in the optimizer step,
// which is fenced by barriers on both sides, so the gather itself needs no handshake.  n % 8 == 0, soff % 8 == 0 (bf16).
__global__ void __launch_bounds__(256)
allgather_pull_kernel(PeerPtrs shards, int world, long long soff, long long n, __nv_bfloat16* __restrict__ out) {
  // 8 independent 16-byte loads per thread per round: a peer load takes a few microseconds over NVLink, so the
  // bandwidth is (bytes in flight) / latency and one load per thread would leave the link idle
  constexpr int U = 8;
  const long long nv = n / 8;
  const long long total = nv * world;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total; i0 += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) {
        const int r = static_cast<int>(i / nv);
        const long long j = i - r * nv;
        v[u] = ld_volatile_u4(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(shards.p[r]) + soff) + j);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < total) reinterpret_cast<uint4*>(out)[i] = v[u];
    }
  }
}

// acc[i] += sum_r ws_r[lo + i]: the per-layer gradient reduction of the parameter-sharded learner (the owner reads its
// slice of every rank's layer workspace, fixed rank order).  n % 4 == 0, lo % 4 == 0.
// MULTIMEM: one `multimem.ld_reduce` through the NVSwitch returns the sum over all ranks (the switch adds), so the owner
// pulls n floats over NVLink instead of world * n.
template <bool MULTIMEM>
__global__ void __launch_bounds__(256)
reduce_scatter_add_kernel(PeerPtrs ws, const float* __restrict__ mc_ws, int world, long long lo, long long n,
                          float* __restrict__ acc) {
  constexpr int U = 4;
  const long long nv = n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nv; i0 += stride * U) {
    float4 a[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      a[u] = i < nv ? reinterpret_cast<const float4*>(acc)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (MULTIMEM) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nv) {
          const float4 x = multimem_ld_reduce_f32x4(mc_ws + lo + i * 4);
          a[u].x += x.x; a[u].y += x.y; a[u].z += x.z; a[u].w += x.w;
        }
      }
    } else
#pragma unroll 1
    for (int r = 0; r < world; ++r) {
      uint4 x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nv) x[u] = ld_volatile_u4(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ws.p[r]) + lo) + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nv) {
          a[u].x += __uint_as_float(x[u].x); a[u].y += __uint_as_float(x[u].y);
          a[u].z += __uint_as_float(x[u].z); a[u].w += __uint_as_float(x[u].w);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nv) reinterpret_cast<float4*>(acc)[i] = a[u];
    }
  }
}

// The same gather by the copy engines: one peer-to-peer copy per rank, no SM involved, so the layer's GEMMs keep the
// whole GPU.  `elem` = bytes per element.
extern "C" int b200_allgather_copy(const void* const* shard_ptrs, int world, long long soff, long long n, int elem,
                                   void* out, void* stream) {
  if (world > MAX_PEERS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  for (int r = 0; r < world; ++r) {
    const char* src = reinterpret_cast<const char*>(shard_ptrs[r]) + soff * elem;
    cudaError_t e = cudaMemcpyAsync(reinterpret_cast<char*>(out) + static_cast<long long>(r) * n * elem, src,
                                    static_cast<size_t>(n) * elem, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return 0;
}

extern "C" int b200_allgather_pull(const void* const* shard_ptrs, int world, long long soff, long long n, void* out,
                                   int ctas, void* stream) {
  if (world > MAX_PEERS || n % 8 || soff % 8) return -1;
  if (n == 0) return 0;
  // a modest grid: the gather runs beside the layer's GEMMs on another stream and must not take the SMs from them
  allgather_pull_kernel<<<ctas > 0 ? ctas : 32, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_ptrs(shard_ptrs, world), world, soff, n, reinterpret_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_reduce_scatter_add(const void* const* ws_ptrs, const void* mc_ws, int world, long long lo, long long n,
                                       float* acc, int ctas, void* stream) {
  if (world > MAX_PEERS || n % 4 || lo % 4) return -1;
  if (n == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (mc_ws)
    reduce_scatter_add_kernel<true><<<ctas > 0 ? ctas : 32, 256, 0, st>>>(make_ptrs(ws_ptrs, world),
                                                                           reinterpret_cast<const float*>(mc_ws), world, lo, n, acc);
  else
    reduce_scatter_add_kernel<false><<<ctas > 0 ? ctas : 32, 256, 0, st>>>(make_ptrs(ws_ptrs, world), nullptr, world, lo, n, acc);
  return static_cast<int>(cudaGetLastError());
}

// out[0 .. n) = sum over ranks of grads_r[lo .. lo+n); sumsq[0] += |out|^2 (the caller zeroes it once per step).
// `ctas` <= 0: a grid that fills the GPU; a smaller grid leaves SMs to kernels running beside it on another stream.
extern "C" int b200_zero_reduce_range(const void* const* grad_ptrs, const void* mc_grads, int world, long long lo,
                                      long long n, float* out, float* sumsq, int use_multimem, int ctas, void* stream) {
  if (world > MAX_PEERS || n % 4 || lo % 4) return -1;
  if (n == 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = ctas > 0 ? ctas : 148 * 4;
  const PeerPtrs pp = make_ptrs(grad_ptrs, world);
  if (use_multimem && mc_grads)
    zero_reduce_scatter_kernel<true, 8, 1><<<grid, 256, 0, st>>>(pp, reinterpret_cast<const float*>(mc_grads), world, lo, n, out, sumsq);
  else if (world <= 2)
    zero_reduce_scatter_kernel<false, 8, 2><<<grid, 256, 0, st>>>(pp, nullptr, world, lo, n, out, sumsq);
  else if (world <= 4)
    zero_reduce_scatter_kernel<false, 4, 4><<<grid, 256, 0, st>>>(pp, nullptr, world, lo, n, out, sumsq);
  else
    zero_reduce_scatter_kernel<false, 2, 8><<<grid, 256, 0, st>>>(pp, nullptr, world, lo, n, out, sumsq);
  return static_cast<int>(cudaGetLastError());
}

// out_shard[n] = sum over ranks of grads_r[lo .. lo+n); sumsq[0] = |out_shard|^2 (overwritten).
extern "C" int b200_zero_reduce_scatter(const void* const* grad_ptrs, const void* mc_grads, int rank, int world,
                                        long long lo, long long n, float* out_shard, float* sumsq, int use_multimem,
                                        void* stream) {
  (void)rank;
  cudaError_t e = cudaMemsetAsync(sumsq, 0, sizeof(float), reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return b200_zero_reduce_range(grad_ptrs, mc_grads, world, lo, n, out_shard, sumsq, use_multimem, 0, stream);
}

extern "C" int b200_zero_adamw_allgather(float* master, float* m, float* v, const float* grad,
                                         const void* const* param_ptrs, void* mc_params, int world, long long goff,
                                         long long n, const float* gscale, float lr, float beta1, float beta2,
                                         float eps, float wd, int step, int use_multimem, void* stream) {
  if (world > MAX_PEERS || n % 8 || goff % 8) return -1;
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = 148 * 8;
  if (use_multimem && mc_params)
    zero_adamw_allgather_kernel<true><<<grid, 256, 0, st>>>(master, m, v, grad, make_ptrs(param_ptrs, world), mc_params,
                                                             world, goff, n, gscale, lr, beta1, beta2, eps, wd, bc1, bc2);
  else
    zero_adamw_allgather_kernel<false><<<grid, 256, 0, st>>>(master, m, v, grad, make_ptrs(param_ptrs, world), nullptr,
                                                              world, goff, n, gscale, lr, beta1, beta2, eps, wd, bc1,
                                                              bc2);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ learner -> engine weight push
// One read of the source slice, one 16-byte store per destination: dst_r[off + i] = src[off + i] for
// every destination r (peer buffers mapped through CUDA IPC or symmetric memory).  With `src_f32`
// the source is the fp32 master copy and the cast to bf16 happens in flight.
namespace b200 {
template <bool F32>
__global__ void __launch_bounds__(256)
multi_push_kernel(const void* __restrict__ src, PeerPtrs dsts, int n_dst, long long off, long long n) {
  const long long nv = n / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 pk;
    if (F32) {
      const float4 a = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + off)[i * 2];
      const float4 b = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + off)[i * 2 + 1];
      pk.x = pack_bf16x2(a.x, a.y); pk.y = pack_bf16x2(a.z, a.w);
      pk.z = pack_bf16x2(b.x, b.y); pk.w = pack_bf16x2(b.z, b.w);
    } else {
      pk = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src) + off)[i];
    }
#pragma unroll 1
    for (int r = 0; r < n_dst; ++r)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dsts.p[r]) + off)[i] = pk;
  }
  // tail (n not a multiple of 8)
  if (blockIdx.x == 0) {
    for (long long i = nv * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const __nv_bfloat16 v = F32 ? __float2bfloat16(reinterpret_cast<const float*>(src)[off + i])
                                  : reinterpret_cast<const __nv_bfloat16*>(src)[off + i];
      for (int r = 0; r < n_dst; ++r) reinterpret_cast<__nv_bfloat16*>(dsts.p[r])[off + i] = v;
    }
  }
  __threadfence_system();
}
}  // namespace b200

// src: bf16 (src_f32 = 0) or fp32 (src_f32 = 1) buffer; copies elements [off, off + n) to the same
// offsets of up to 8 destination bf16 buffers.  `off` must be a multiple of 8.
extern "C" int b200_multi_push(const void* src, const void* const* dst_ptrs, int n_dst, long long off, long long n, int src_f32,
                               void* stream) {
  if (n <= 0 || n_dst <= 0) return 0;
  if (n_dst > MAX_PEERS || off % 8) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (src_f32) multi_push_kernel<true><<<148 * 8, 256, 0, st>>>(src, make_ptrs(dst_ptrs, n_dst), n_dst, off, n);
  else multi_push_kernel<false><<<148 * 8, 256, 0, st>>>(src, make_ptrs(dst_ptrs, n_dst), n_dst, off, n);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ learner -> tensor-parallel engine weight push
// The engines' ranks hold SHARDS of every layer in their own flat layout (q/k/v and gate/up rows, o_proj / down_proj columns
// of their heads and channels; embedding, head and norms whole).  Instead of sending every rank the full model and letting
// it re-shard (twice the bytes at TP = 2 and one more pass over the engine's memory), the learner's kernel writes every
// piece straight to its place: the host describes the re-layout once as a table of 2-D copy tiles
// (``parallel/weight_sync.py:tp_push_plan``), each with a bit mask of the destination buffers that receive it.
namespace b200 {
struct PushTile {
  long long src;         // element offset in the source buffer
  long long dst;         // element offset in every destination buffer of the mask
  long long src_stride;  // elements between consecutive rows in the source
  long long dst_stride;  // ... in the destination
  int rows, row_len;     // rows x elements per row
  unsigned mask;         // bit d set: destination d receives this tile
  int pad_;
};

template <bool F32>
__global__ void __launch_bounds__(256)
tp_push_kernel(const void* __restrict__ src, PeerPtrs dsts, int n_dst, const PushTile* __restrict__ tiles, int n_tiles) {
  for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const PushTile tl = tiles[t];
    const bool vec = ((tl.src | tl.dst | tl.src_stride | tl.dst_stride | tl.row_len) & 7) == 0;
    if (vec) {
      const int nvr = tl.row_len >> 3;
      const long long total = static_cast<long long>(tl.rows) * nvr;
      for (long long i = threadIdx.x; i < total; i += blockDim.x) {
        const long long r = i / nvr, c = i - r * nvr;
        const long long so = tl.src + r * tl.src_stride + c * 8, d_o = tl.dst + r * tl.dst_stride + c * 8;
        uint4 pk;
        if (F32) {
          const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + so);
          const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + so + 4);
          pk.x = pack_bf16x2(a.x, a.y); pk.y = pack_bf16x2(a.z, a.w);
          pk.z = pack_bf16x2(b.x, b.y); pk.w = pack_bf16x2(b.z, b.w);
        } else {
          pk = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src) + so);
        }
#pragma unroll 1
        for (int d = 0; d < n_dst; ++d)
          if (tl.mask >> d & 1u) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dsts.p[d]) + d_o) = pk;
      }
    } else {
      const long long total = static_cast<long long>(tl.rows) * tl.row_len;
      for (long long i = threadIdx.x; i < total; i += blockDim.x) {
        const long long r = i / tl.row_len, c = i - r * tl.row_len;
        const long long so = tl.src + r * tl.src_stride + c, d_o = tl.dst + r * tl.dst_stride + c;
        const __nv_bfloat16 v = F32 ? __float2bfloat16(reinterpret_cast<const float*>(src)[so]) : reinterpret_cast<const __nv_bfloat16*>(src)[so];
        for (int d = 0; d < n_dst; ++d)
          if (tl.mask >> d & 1u) reinterpret_cast<__nv_bfloat16*>(dsts.p[d])[d_o] = v;
      }
    }
  }
  __threadfence_system();
}
}  // namespace b200

// src: bf16 (src_f32 = 0) or fp32 buffer of the learner; dst_ptrs: up to 8 destination bf16 buffers (engine e, rank r at
// index e * tp + r); tiles: device array of `n_tiles` PushTile records.
extern "C" int b200_tp_push(const void* src, const void* const* dst_ptrs, int n_dst, const void* tiles, int n_tiles, int src_f32,
                            void* stream) {
  if (n_tiles <= 0 || n_dst <= 0) return 0;
  if (n_dst > MAX_PEERS) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = n_tiles < 148 * 8 ? n_tiles : 148 * 8;
  const PushTile* tp = reinterpret_cast<const PushTile*>(tiles);
  if (src_f32) tp_push_kernel<true><<<grid, 256, 0, st>>>(src, make_ptrs(dst_ptrs, n_dst), n_dst, tp, n_tiles);
  else tp_push_kernel<false><<<grid, 256, 0, st>>>(src, make_ptrs(dst_ptrs, n_dst), n_dst, tp, n_tiles);
  return static_cast<int>(cudaGetLastError());
}

// Lets kernels running on `dev` dereference pointers into `peer`'s memory (needed before a kernel writes through a
// CUDA-IPC mapping of another GPU's buffer; copies issued by the runtime enable it on their own, raw kernels do not).
// Returns 0 on success or if access was already enabled, 1 if the two devices cannot reach each other, else the CUDA error.
extern "C" int b200_enable_peer_access(int dev, int peer) {
  if (dev == peer) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, dev, peer);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (!can) return 1;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(dev);
  e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
  cudaSetDevice(prev);
  return static_cast<int>(e);
}

// ---------------------------------------------------------------------------------------------------------------
// Cross-process buffer sharing for the weight push.  The exporting process describes the allocation that contains
// `ptr` (64-byte IPC handle + byte offset of `ptr` inside it); the importing process opens the handle WITH ITS OWN
// COMPUTE DEVICE CURRENT, so the mapping is created in the address space of the device whose kernels will store
// through it (an IPC mapping belongs to the context that opened it; peer access to the exporting GPU is switched on
// by the open itself via the lazy-peer-access flag).
// ---------------------------------------------------------------------------------------------------------------
typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

extern "C" int b200_ipc_export(const void* ptr, unsigned char* handle_out, long long* offset_out, long long* size_out) {
  static GetAddressRangeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<GetAddressRangeFn>(p);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return -2;
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle_out, &h, 64);
  *offset_out = static_cast<long long>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  *size_out = static_cast<long long>(size);
  return 0;
}

// Opens the handle with device `dev` current; *base_out is the mapped base of the exporter's allocation.
extern "C" int b200_ipc_open(int dev, const unsigned char* handle, void** base_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(dev);
  cudaError_t e = cudaIpcOpenMemHandle(base_out, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) cudaGetLastError();
  cudaSetDevice(prev);
  return static_cast<int>(e);
}

extern "C" int b200_ipc_close(int dev, void* base) {
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(dev);
  cudaError_t e = cudaIpcCloseMemHandle(base);
  if (e != cudaSuccess) cudaGetLastError();
  cudaSetDevice(prev);
  return static_cast<int>(e);
}
