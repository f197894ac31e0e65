// Memory-bound kernels of the decoder layer and the optimizer, written for HBM3e streaming:
// 16-byte vector accesses, one pass over each tensor, fp32 math, bf16 storage.
//   RMSNorm fwd/bwd (with fused residual add), RoPE (in place on fused QKV, per-document
//   positions), SwiGLU fwd/bwd on fused gate|up, embedding gather / scatter-add,
//   sum-of-squares (grad norm), partitioned AdamW with bf16 shard refresh, casts.
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum; `red` is >= 32 floats of shared memory; result broadcast to all threads
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

// ------------------------------------------------------------------ RMSNorm forward
// h = x (+ res);  y = h * rsqrt(mean(h^2) + eps) * w.  Writes h back to `h_out` when a
// residual is given (the new residual stream), rstd[row] for the backward.
// X32: x is an fp32 accumulator (split-K GEMM output) that is consumed here: it is read, zeroed for the next GEMM that adds
// into it, and rounded to bf16 before the residual is added (what a bf16 GEMM output would have been).
// X32 with nparts > 0: x is `nparts` fp32 planes `part_stride` floats apart (the K slices of a split-K GEMM written with
// plain stores); they are summed in plane order and nothing is zeroed.
template <bool X32>
__global__ void rmsnorm_fwd_kernel(const void* __restrict__ x_any, const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int D, float eps, int nparts = 0,
                                   long long part_stride = 0) {
  griddep_launch_dependents();  // the decode GEMM that follows may bring its first weight tiles in while this kernel runs
  griddep_wait();               // launched with programmatic serialization: the input is the predecessor's output
  __shared__ float red[32];
  extern __shared__ __align__(16) uint8_t dyn[];
  float* hbuf = reinterpret_cast<float*>(dyn);  // D floats: keeps h so x is read once
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(reinterpret_cast<const __nv_bfloat16*>(x_any) + row * D);
  float4* x32 = reinterpret_cast<float4*>(const_cast<float*>(reinterpret_cast<const float*>(x_any)) + row * D);
  const bf16x8* rr = res ? reinterpret_cast<const bf16x8*>(res + row * D) : nullptr;
  const int nv = D / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float f[8];
    if (X32) {
      float4 a = x32[2 * i], b = x32[2 * i + 1];
      if (nparts == 0) {
        x32[2 * i] = make_float4(0.f, 0.f, 0.f, 0.f);
        x32[2 * i + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      for (int p = 1; p < nparts; ++p) {
        const float4* xp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x_any) + p * part_stride + row * D);
        const float4 a2 = xp[2 * i], b2 = xp[2 * i + 1];
        a.x += a2.x; a.y += a2.y; a.z += a2.z; a.w += a2.w;
        b.x += b2.x; b.y += b2.y; b.z += b2.z; b.w += b2.w;
      }
      const float t[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16(t[j]));
    } else {
      unpack8(xr[i], f);
    }
    if (rr) {
      float g[8];
      unpack8(rr[i], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      bf16x8 p = pack8(f);
      reinterpret_cast<bf16x8*>(h_out + row * D)[i] = p;
      unpack8(p, f);  // normalise the rounded residual stream, as an unfused add would
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ss += f[j] * f[j];
      hbuf[i * 8 + j] = f[j];
    }
  }
  const float tot = block_sum(ss, red);
  const float r = rsqrtf(tot / D + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float wf[8], o[8];
    unpack8(wr[i], wf);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // match the reference module order: (h * rstd) rounded to bf16, then * weight
      const float n = __bfloat162float(__float2bfloat16(hbuf[i * 8 + j] * r));
      o[j] = n * wf[j];
    }
    reinterpret_cast<bf16x8*>(y + row * D)[i] = pack8(o);
  }
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = rstd * (g - xhat * mean(g * xhat)) (+ dres), g = dy * w, xhat = h * rstd.
// dw partial sums go to `dw_partial[blockIdx.x][D]` (scratch), reduced by rmsnorm_dw_reduce.
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w,
                                   const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int T, int D) {
  __shared__ float red[32];
  extern __shared__ __align__(16) uint8_t dyn[];
  float* dwacc = reinterpret_cast<float*>(dyn);  // D floats per CTA
  for (int i = threadIdx.x; i < D; i += blockDim.x) dwacc[i] = 0.f;
  const int nv = D / 8;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + row * D);
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * D);
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float hf[8], df[8], wf[8];
      unpack8(hr[i], hf);
      unpack8(dyr[i], df);
      unpack8(wr[i], wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += df[j] * wf[j] * hf[j] * r;
    }
    const float mean_gx = block_sum(dot, red) / D;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float hf[8], df[8], wf[8], o[8];
      unpack8(hr[i], hf);
      unpack8(dyr[i], df);
      unpack8(wr[i], wf);
      float rf[8];
      if (dres) unpack8(reinterpret_cast<const bf16x8*>(dres + row * D)[i], rf);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = hf[j] * r;
        o[j] = r * (df[j] * wf[j] - xhat * mean_gx);
        if (dres) o[j] += rf[j];
        dwacc[i * 8 + j] += df[j] * xhat;  // same thread owns column i*8+j for every row
      }
      reinterpret_cast<bf16x8*>(dx + row * D)[i] = pack8(o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) dw_partial[static_cast<long long>(blockIdx.x) * D + i] = dwacc[i];
}

// The same backward for D = 2048 * VPT: every thread keeps its VPT 16-byte vectors of h and dy in registers (one read
// of each row, no second pass), its weight-gradient partial sums too, and issues the NEXT row's loads before the block
// reduction of the current one, so that the memory latency overlaps the reduction instead of adding to it.
template <int VPT>
__global__ void __launch_bounds__(256, VPT <= 2 ? 2 : 1)
rmsnorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w,
                       const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dy,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw_partial, int T) {
  constexpr int D = 2048 * VPT;
  __shared__ float red[32];
  float wf[VPT][8], dwr[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    unpack8(reinterpret_cast<const bf16x8*>(w)[threadIdx.x + v * 256], wf[v]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dwr[v][j] = 0.f;
  }
  bf16x8 hv[VPT], dv[VPT], rv[VPT], hn[VPT], dn[VPT], rn[VPT];
  long long row = blockIdx.x;
  if (row < T) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      hv[v] = reinterpret_cast<const bf16x8*>(h + row * D)[threadIdx.x + v * 256];
      dv[v] = reinterpret_cast<const bf16x8*>(dy + row * D)[threadIdx.x + v * 256];
      if (dres) rv[v] = reinterpret_cast<const bf16x8*>(dres + row * D)[threadIdx.x + v * 256];
    }
  }
  for (; row < T; row += gridDim.x) {
    const long long nrow = row + gridDim.x;
    if (nrow < T) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        hn[v] = reinterpret_cast<const bf16x8*>(h + nrow * D)[threadIdx.x + v * 256];
        dn[v] = reinterpret_cast<const bf16x8*>(dy + nrow * D)[threadIdx.x + v * 256];
        if (dres) rn[v] = reinterpret_cast<const bf16x8*>(dres + nrow * D)[threadIdx.x + v * 256];
      }
    }
    const float r = rstd[row];
    float hf[VPT][8], df[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      unpack8(hv[v], hf[v]);
      unpack8(dv[v], df[v]);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += df[v][j] * wf[v][j] * hf[v][j] * r;
    }
    const float mean_gx = block_sum(dot, red) / D;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      float o[8], rf[8];
      if (dres) unpack8(rv[v], rf);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xhat = hf[v][j] * r;
        o[j] = r * (df[v][j] * wf[v][j] - xhat * mean_gx);
        if (dres) o[j] += rf[j];
        dwr[v][j] += df[v][j] * xhat;
      }
      reinterpret_cast<bf16x8*>(dx + row * D)[threadIdx.x + v * 256] = pack8(o);
    }
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      hv[v] = hn[v];
      dv[v] = dn[v];
      rv[v] = rn[v];
    }
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v)
#pragma unroll
    for (int j = 0; j < 8; ++j)
      dw_partial[static_cast<long long>(blockIdx.x) * D + (threadIdx.x + v * 256) * 8 + j] = dwr[v][j];
}

// dw_out[d] += sum_p partial[p][d]   (fp32 main-grad accumulate).  A CTA of 32 x 8 threads owns 32 columns: the eight
// thread rows walk interleaved partial rows (128-byte coalesced loads), then add up through shared memory in a fixed
// order.  (One thread per column walking all P rows took 23 us for P = 296: a chain of dependent-latency loads.)
__global__ void __launch_bounds__(256)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw_out, int P, int D) {
  __shared__ float red[8][32];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int d = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (d < D)
    for (int p = ty; p < P; p += 8) s += partial[static_cast<long long>(p) * D + d];
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && d < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][tx];
    dw_out[d] += t;
  }
}

// ------------------------------------------------------------------ RoPE
// In place on fused qkv [T, (Hq + 2*Hkv) * Dh]; rotates the Hq query heads and Hkv key heads
// with the half-split convention: out[i] = x[i]*cos - x[i+h]*sin, out[i+h] = x[i+h]*cos + x[i]*sin.
// `inv_freq` [Dh/2] carries any frequency scaling; `sign` = +1 forward, -1 backward (transpose).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                            const float* __restrict__ inv_freq, int T, int Hq, int Hkv, int Dh, float sign) {
  const int half = Dh / 2;
  const int heads = Hq + Hkv;
  const long long row_stride = static_cast<long long>(Hq + 2 * Hkv) * Dh;
  const long long total = static_cast<long long>(T) * heads * (half / 2);  // 2 pairs per thread
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int p2 = static_cast<int>(idx % (half / 2));
    const long long th = idx / (half / 2);
    const int hd = static_cast<int>(th % heads);
    const long long t = th / heads;
    const float ps = static_cast<float>(pos[t]);
    __nv_bfloat16* base = qkv + t * row_stride + static_cast<long long>(hd) * Dh;
    const int i = p2 * 2;
    __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(base + i);
    __nv_bfloat162 hi = *reinterpret_cast<__nv_bfloat162*>(base + i + half);
    float2 l = __bfloat1622float2(lo), h = __bfloat1622float2(hi);
    float s0, c0, s1, c1;
    sincosf(ps * inv_freq[i], &s0, &c0);
    sincosf(ps * inv_freq[i + 1], &s1, &c1);
    s0 *= sign;
    s1 *= sign;
    float2 ol = make_float2(l.x * c0 - h.x * s0, l.y * c1 - h.y * s1);
    float2 oh = make_float2(h.x * c0 + l.x * s0, h.y * c1 + l.y * s1);
    *reinterpret_cast<__nv_bfloat162*>(base + i) = __floats2bfloat162_rn(ol.x, ol.y);
    *reinterpret_cast<__nv_bfloat162*>(base + i + half) = __floats2bfloat162_rn(oh.x, oh.y);
  }
}

// Rotation table for one packed batch: tab[t][i] = (cos, sin)(pos[t] * inv_freq[i]).  Computed once per micro-batch and
// reused by every layer's forward and backward rotation (sincosf is by far the most expensive part of the rotation).
__global__ void rope_table_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq, float2* __restrict__ tab, long long T,
                                  int half) {
  const long long total = T * half;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    float s, c;
    sincosf(static_cast<float>(pos[idx / half]) * inv_freq[idx % half], &s, &c);
    tab[idx] = make_float2(c, s);
  }
}

// Rotation from the table: one thread rotates 8 (lo, hi) pairs of one head with 16-byte accesses.  Dh % 16 == 0.
__global__ void rope_apply_kernel(__nv_bfloat16* __restrict__ qkv, const float2* __restrict__ tab, long long T, int Hq, int Hkv, int Dh,
                                  float sign) {
  griddep_launch_dependents();
  griddep_wait();
  const int half = Dh / 2, nchunk = half / 8, heads = Hq + Hkv;
  const long long row_stride = static_cast<long long>(Hq + 2 * Hkv) * Dh;
  const long long total = T * heads * nchunk;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % nchunk);
    const long long th = idx / nchunk;
    const int hd = static_cast<int>(th % heads);
    const long long t = th / heads;
    __nv_bfloat16* base = qkv + t * row_stride + static_cast<long long>(hd) * Dh + c * 8;
    float lo[8], hi[8], ol[8], oh[8];
    unpack8(*reinterpret_cast<const bf16x8*>(base), lo);
    unpack8(*reinterpret_cast<const bf16x8*>(base + half), hi);
    const float4* tv = reinterpret_cast<const float4*>(tab + t * half + c * 8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 cs = tv[j];  // (cos, sin) of pairs 2j and 2j + 1
      const float s0 = cs.y * sign, s1 = cs.w * sign;
      ol[2 * j] = lo[2 * j] * cs.x - hi[2 * j] * s0;
      oh[2 * j] = hi[2 * j] * cs.x + lo[2 * j] * s0;
      ol[2 * j + 1] = lo[2 * j + 1] * cs.z - hi[2 * j + 1] * s1;
      oh[2 * j + 1] = hi[2 * j + 1] * cs.z + lo[2 * j + 1] * s1;
    }
    *reinterpret_cast<bf16x8*>(base) = pack8(ol);
    *reinterpret_cast<bf16x8*>(base + half) = pack8(oh);
  }
}

// ------------------------------------------------------------------ SwiGLU
// gate_up [T, 2F] (gate | up) -> act [T, F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, long long T,
                                  int F) {
  griddep_launch_dependents();  // see rmsnorm_fwd_kernel
  griddep_wait();
  const int nv = F / 8;
  const long long total = T * nv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / nv;
    const int i = static_cast<int>(idx % nv);
    float g[8], u[8], o[8];
    unpack8(reinterpret_cast<const bf16x8*>(gu + t * 2 * F)[i], g);
    unpack8(reinterpret_cast<const bf16x8*>(gu + t * 2 * F + F)[i], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<bf16x8*>(act + t * F)[i] = pack8(o);
  }
}
// dgu [T, 2F] from dact [T, F]; may alias gu (in place) since each thread reads before writing.
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* gu, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* dgu, long long T, int F) {
  const int nv = F / 8;
  const long long total = T * nv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / nv;
    const int i = static_cast<int>(idx % nv);
    float g[8], u[8], d[8], og[8], ou[8];
    unpack8(reinterpret_cast<const bf16x8*>(gu + t * 2 * F)[i], g);
    unpack8(reinterpret_cast<const bf16x8*>(gu + t * 2 * F + F)[i], u);
    unpack8(reinterpret_cast<const bf16x8*>(dact + t * F)[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * s;
      og[j] = d[j] * u[j] * (s + silu * (1.f - s));
      ou[j] = d[j] * silu;
    }
    reinterpret_cast<bf16x8*>(dgu + t * 2 * F)[i] = pack8(og);
    reinterpret_cast<bf16x8*>(dgu + t * 2 * F + F)[i] = pack8(ou);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ ids,
                                     __nv_bfloat16* __restrict__ out, int T, int D, int V) {
  const int nv = D / 8;
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    long long id = ids[row];
    if (id < 0 || id >= V) id = 0;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(table + id * D);
    bf16x8* dst = reinterpret_cast<bf16x8*>(out + row * D);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = src[i];
  }
}
// grad_table[ids[t]] += dout[t]   (fp32 atomics: several tokens may share an id)
__global__ void embedding_bwd_kernel(float* __restrict__ grad_table, const long long* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ dout, int T, int D, int V) {
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const long long id = ids[row];
    if (id < 0 || id >= V) continue;
    for (int i = threadIdx.x; i < D; i += blockDim.x)
      atomicAdd(grad_table + id * D + i, __bfloat162float(dout[row * D + i]));
  }
}

// ------------------------------------------------------------------ sum of squares
// partial[blockIdx.x] = sum over this CTA's grid-stride slice of g^2; finalised by sumsq_final.
__global__ void sumsq_partial_kernel(const float* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const long long nv = n / 4;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = g4[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = nv * 4 + threadIdx.x; i < n; i += blockDim.x) s += g[i] * g[i];
  const float tot = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = tot;
}
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int P, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += partial[i];
  const float tot = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + tot : tot;
}

// ------------------------------------------------------------------ AdamW on an fp32 shard
// g = grad * gscale[0] (device scalar: clip coefficient / accumulation divisor);
// decoupled weight decay; writes the refreshed bf16 working copy; optionally zeroes the grad.
__device__ __forceinline__ float adamw_one(float& p, float& mi, float& vi, float g, float lr, float beta1, float beta2, float eps, float wd,
                                           float bc1, float bc2) {
  mi = beta1 * mi + (1.f - beta1) * g;
  vi = beta2 * vi + (1.f - beta2) * g * g;
  p *= (1.f - lr * wd);
  p -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
  return p;
}

// VEC: every pointer is 16-byte aligned (8 for the bf16 copy): four elements per thread and iteration, 16-byte accesses.
template <bool VEC>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, float* __restrict__ grad,
             __nv_bfloat16* __restrict__ param_bf16, long long n, const float* __restrict__ gscale, float lr, float beta1, float beta2,
             float eps, float wd, float bc1, float bc2, int zero_grad) {
  const float gs = gscale ? gscale[0] : 1.f;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  long long done = 0;
  if (VEC) {
    const long long nv = n / 4;
    for (long long i = tid; i < nv; i += nthreads) {
      const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
      float4 p4 = reinterpret_cast<const float4*>(master)[i];
      float4 m4 = reinterpret_cast<const float4*>(m)[i];
      float4 v4 = reinterpret_cast<const float4*>(v)[i];
      adamw_one(p4.x, m4.x, v4.x, g4.x * gs, lr, beta1, beta2, eps, wd, bc1, bc2);
      adamw_one(p4.y, m4.y, v4.y, g4.y * gs, lr, beta1, beta2, eps, wd, bc1, bc2);
      adamw_one(p4.z, m4.z, v4.z, g4.z * gs, lr, beta1, beta2, eps, wd, bc1, bc2);
      adamw_one(p4.w, m4.w, v4.w, g4.w * gs, lr, beta1, beta2, eps, wd, bc1, bc2);
      reinterpret_cast<float4*>(m)[i] = m4;
      reinterpret_cast<float4*>(v)[i] = v4;
      reinterpret_cast<float4*>(master)[i] = p4;
      if (param_bf16) reinterpret_cast<uint2*>(param_bf16)[i] = make_uint2(pack_bf16x2(p4.x, p4.y), pack_bf16x2(p4.z, p4.w));
      if (zero_grad) reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    done = nv * 4;
  }
  for (long long i = done + tid; i < n; i += nthreads) {
    float p = master[i], mi = m[i], vi = v[i];
    adamw_one(p, mi, vi, grad[i] * gs, lr, beta1, beta2, eps, wd, bc1, bc2);
    m[i] = mi;
    v[i] = vi;
    master[i] = p;
    if (param_bf16) param_bf16[i] = __float2bfloat16(p);
    if (zero_grad) grad[i] = 0.f;
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                                        float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16(src[i] * scale);
}
__global__ void axpy_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] += __bfloat162float(src[i]);
}

static inline int grid_for(long long work, int threads, int cap = 148 * 16) {
  long long g = (work + threads - 1) / threads;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace b200

using namespace b200;
#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<__nv_bfloat16*>(p)
#define CBF(p) reinterpret_cast<const __nv_bfloat16*>(p)

extern "C" int b200_rmsnorm_fwd(const void* x, const void* res, const void* w, void* h_out, void* y, float* rstd,
                                int T, int D, float eps, void* stream) {
  if (T <= 0) return 0;
  if (D % 8) return -1;
  const int threads = D >= 2048 ? 256 : 128;
  static std::atomic<unsigned long long> cfg{0};
  {
    cudaError_t e = opt_in_shared_memory(rmsnorm_fwd_kernel<false>, 64 * 1024, cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  if (D * 4 > 64 * 1024) return -2;
  cudaError_t le = launch_pdl(rmsnorm_fwd_kernel<false>, dim3(T), dim3(threads), D * sizeof(float), ST(stream), x, CBF(res), CBF(w), BF(h_out),
                              BF(y), rstd, D, eps, 0, 0LL);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}

// Same, with x an fp32 [T, D] accumulator that is consumed (read, then zeroed): the partner of the split-K GEMM.
extern "C" int b200_rmsnorm_fwd_acc32(float* x32, const void* res, const void* w, void* h_out, void* y, float* rstd, int T, int D,
                                      float eps, void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || D * 4 > 64 * 1024) return -1;
  const int threads = D >= 2048 ? 256 : 128;
  static std::atomic<unsigned long long> cfg{0};
  {
    cudaError_t e = opt_in_shared_memory(rmsnorm_fwd_kernel<true>, 64 * 1024, cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaError_t le = launch_pdl(rmsnorm_fwd_kernel<true>, dim3(T), dim3(threads), D * sizeof(float), ST(stream), static_cast<const void*>(x32),
                              CBF(res), CBF(w), BF(h_out), BF(y), rstd, D, eps, 0, 0LL);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}

// Same, with x given as `nparts` fp32 planes [nparts][T][D] (`part_stride` floats apart) that are summed, not zeroed: the
// partner of the K-split decode GEMM, which writes one plane per K slice with plain stores.
extern "C" int b200_rmsnorm_fwd_parts(const float* x32, int nparts, long long part_stride, const void* res, const void* w, void* h_out,
                                      void* y, int T, int D, float eps, void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || D * 4 > 64 * 1024 || nparts < 1) return -1;
  const int threads = D >= 2048 ? 256 : 128;
  static std::atomic<unsigned long long> cfg{0};
  {
    cudaError_t e = opt_in_shared_memory(rmsnorm_fwd_kernel<true>, 64 * 1024, cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaError_t le = launch_pdl(rmsnorm_fwd_kernel<true>, dim3(T), dim3(threads), D * sizeof(float), ST(stream), static_cast<const void*>(x32),
                              CBF(res), CBF(w), BF(h_out), BF(y), static_cast<float*>(nullptr), D, eps, nparts, part_stride);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}

// Shared by both entry points: picks the register-resident kernel where D allows it, launches it with at most `max_ctas`
// CTAs (`dw_partial` has that many rows of D floats) and reduces the partial rows into `dw_out`.
static void launch_rmsnorm_bwd(const void* h, const void* w, const float* rstd, const void* dy, const void* dres, void* dx,
                               float* dw_partial, float* dw_out, int T, int D, int max_ctas, cudaStream_t st) {
  int ctas = T < max_ctas ? T : max_ctas;
  if (D == 2048 || D == 4096 || D == 8192) {
    // two resident CTAs per SM (one at D = 8192), each with the next row's loads in flight
    const int cap = D == 8192 ? 148 : 296;
    if (ctas > cap) ctas = cap;
    if (D == 2048)
      rmsnorm_bwd_reg_kernel<1><<<ctas, 256, 0, st>>>(CBF(h), CBF(w), rstd, CBF(dy), CBF(dres), BF(dx), dw_partial, T);
    else if (D == 4096)
      rmsnorm_bwd_reg_kernel<2><<<ctas, 256, 0, st>>>(CBF(h), CBF(w), rstd, CBF(dy), CBF(dres), BF(dx), dw_partial, T);
    else
      rmsnorm_bwd_reg_kernel<4><<<ctas, 256, 0, st>>>(CBF(h), CBF(w), rstd, CBF(dy), CBF(dres), BF(dx), dw_partial, T);
  } else {
    // blockDim * 8 must cover whole vectors consistently: thread i owns vectors i, i+blockDim, ...
    rmsnorm_bwd_kernel<<<ctas, 256, D * sizeof(float), st>>>(CBF(h), CBF(w), rstd, CBF(dy), CBF(dres), BF(dx), dw_partial, T, D);
  }
  if (dw_out) rmsnorm_dw_reduce_kernel<<<(D + 31) / 32, 256, 0, st>>>(dw_partial, dw_out, ctas, D);
}

// number of partial rows the backward needs in its scratch buffer ([ctas, D] floats)
// four CTAs per SM: one CTA walks its rows one at a time (two block reductions per row), so rows in flight = CTAs
extern "C" int b200_rmsnorm_bwd_ctas(int T) { return T < 592 ? T : 592; }

extern "C" int b200_rmsnorm_bwd(const void* h, const void* w, const float* rstd, const void* dy, const void* dres,
                                void* dx, float* dw_partial, float* dw_out, int T, int D, void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || D * 4 > 64 * 1024) return -1;
  static std::atomic<unsigned long long> cfg{0};
  {
    cudaError_t e = opt_in_shared_memory(rmsnorm_bwd_kernel, 64 * 1024, cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  launch_rmsnorm_bwd(h, w, rstd, dy, dres, dx, dw_partial, dw_out, T, D, b200_rmsnorm_bwd_ctas(T), ST(stream));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_rope(void* qkv, const int* pos, const float* inv_freq, int T, int Hq, int Hkv, int Dh, int backward,
                         void* stream) {
  if (T <= 0) return 0;
  if (Dh % 4) return -1;
  const long long total = static_cast<long long>(T) * (Hq + Hkv) * (Dh / 4);
  rope_kernel<<<grid_for(total, 256), 256, 0, ST(stream)>>>(BF(qkv), pos, inv_freq, T, Hq, Hkv, Dh,
                                                            backward ? -1.f : 1.f);
  return static_cast<int>(cudaGetLastError());
}

// table [T, Dh/2] float2 (cos, sin)
extern "C" int b200_rope_table(const int* pos, const float* inv_freq, void* table, int T, int Dh, void* stream) {
  if (T <= 0) return 0;
  const long long total = static_cast<long long>(T) * (Dh / 2);
  rope_table_kernel<<<grid_for(total, 256), 256, 0, ST(stream)>>>(pos, inv_freq, reinterpret_cast<float2*>(table), T, Dh / 2);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_rope_apply(void* qkv, const void* table, int T, int Hq, int Hkv, int Dh, int backward, void* stream) {
  if (T <= 0) return 0;
  if (Dh % 16) return -1;
  const long long total = static_cast<long long>(T) * (Hq + Hkv) * (Dh / 16);
  cudaError_t le = launch_pdl(rope_apply_kernel, dim3(grid_for(total, 256)), dim3(256), 0, ST(stream), BF(qkv), reinterpret_cast<const float2*>(table),
                              static_cast<long long>(T), Hq, Hkv, Dh, backward ? -1.f : 1.f);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}

extern "C" int b200_swiglu_fwd(const void* gu, void* act, long long T, int F, void* stream) {
  if (T <= 0) return 0;
  if (F % 8) return -1;
  cudaError_t le = launch_pdl(swiglu_fwd_kernel, dim3(grid_for(T * (F / 8), 256)), dim3(256), 0, ST(stream), CBF(gu), BF(act), T, F);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}
extern "C" int b200_swiglu_bwd(const void* gu, const void* dact, void* dgu, long long T, int F, void* stream) {
  if (T <= 0) return 0;
  if (F % 8) return -1;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, ST(stream)>>>(CBF(gu), CBF(dact), BF(dgu), T, F);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_embedding_fwd(const void* table, const long long* ids, void* out, int T, int D, int V,
                                  void* stream) {
  if (T <= 0) return 0;
  if (D % 8) return -1;
  embedding_fwd_kernel<<<T < 4096 ? T : 4096, 128, 0, ST(stream)>>>(CBF(table), ids, BF(out), T, D, V);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int b200_embedding_bwd(float* grad_table, const long long* ids, const void* dout, int T, int D, int V,
                                  void* stream) {
  if (T <= 0) return 0;
  embedding_bwd_kernel<<<T < 4096 ? T : 4096, 256, 0, ST(stream)>>>(grad_table, ids, CBF(dout), T, D, V);
  return static_cast<int>(cudaGetLastError());
}

// scratch: >= 1184 floats. out[0] (=|+=) sum(g^2).
extern "C" int b200_sumsq_scratch_floats() { return 148 * 8; }
extern "C" int b200_sumsq(const float* g, long long n, float* scratch, float* out, int accumulate, void* stream) {
  const int P = n <= 0 ? 1 : grid_for((n + 3) / 4, 256, 148 * 8);
  if (n <= 0) {
    if (!accumulate) cudaMemsetAsync(out, 0, sizeof(float), ST(stream));
    return static_cast<int>(cudaGetLastError());
  }
  sumsq_partial_kernel<<<P, 256, 0, ST(stream)>>>(g, n, scratch);
  sumsq_final_kernel<<<1, 256, 0, ST(stream)>>>(scratch, P, out, accumulate);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_adamw(float* master, float* m, float* v, float* grad, void* param_bf16, long long n,
                          const float* gscale, float lr, float beta1, float beta2, float eps, float wd, int step,
                          int zero_grad, void* stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  const uintptr_t bits = reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(grad) | (reinterpret_cast<uintptr_t>(param_bf16) << 1);
  if ((bits & 15) == 0)
    adamw_kernel<true><<<grid_for(n / 4 + 1, 256, 148 * 8), 256, 0, ST(stream)>>>(master, m, v, grad, BF(param_bf16), n, gscale, lr, beta1, beta2,
                                                                                   eps, wd, bc1, bc2, zero_grad);
  else
    adamw_kernel<false><<<grid_for(n, 256, 148 * 8), 256, 0, ST(stream)>>>(master, m, v, grad, BF(param_bf16), n, gscale, lr, beta1, beta2, eps,
                                                                            wd, bc1, bc2, zero_grad);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_cast_f32_bf16(const float* src, void* dst, long long n, float scale, void* stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(src, BF(dst), n, scale);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int b200_accum_bf16_f32(const void* src, float* dst, long long n, void* stream) {
  if (n <= 0) return 0;
  axpy_bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(CBF(src), dst, n);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ allocation-free RMSNorm backward
// See no_alloc.h.  The per-CTA weight-gradient partials, which b200_rmsnorm_bwd takes from the
// caller, live here in a fixed array that is part of the loaded module.
namespace b200 {
constexpr int NOALLOC_MAX_D = 8192;
constexpr int NOALLOC_MAX_CTAS = 296;
static __device__ __align__(256) float g_rmsnorm_bwd_partials[NOALLOC_MAX_CTAS * NOALLOC_MAX_D];
// Device address of the array above, per device ordinal.  In host code the array's name is only
// a handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress.
static float* g_partials_addr[64] = {nullptr};
}  // namespace b200

extern "C" int b200_rmsnorm_bwd_noalloc_max_d() { return b200::NOALLOC_MAX_D; }

extern "C" int b200_rmsnorm_bwd_noalloc(const void* h, const void* w, const float* rstd, const void* dy,
                                        const void* dres, void* dx, float* dw_out, int T, int D, void* stream) {
  if (T <= 0) return 0;
  if (D % 8 || D <= 0) return -1;
  if (D > NOALLOC_MAX_D) {
    fprintf(stderr, "b200_rmsnorm_bwd_noalloc: D=%d exceeds the built-in scratch (max D %d); use b200_rmsnorm_bwd\n", D,
            NOALLOC_MAX_D);
    return -3;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return -4;
  if (!g_partials_addr[dev]) {
    // first call on this device (it is the current one): resolve the array and opt in to the
    // kernel's dynamic shared memory.  Neither call allocates.
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_bwd_partials);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_partials_addr[dev] = p;
  }
  float* partials = g_partials_addr[dev];
  // every CTA overwrites its whole [D] row of the partials, so nothing left by an earlier call is read
  launch_rmsnorm_bwd(h, w, rstd, dy, dres, dx, partials, dw_out, T, D, NOALLOC_MAX_CTAS, ST(stream));
  return static_cast<int>(cudaGetLastError());
}
