// Token log-probabilities from bf16 logits without an fp32 [T, V] tensor.
//
//   forward : one streaming pass per row with an online softmax: lse, log p(label), entropy
//   backward: rewrites the same bf16 logits buffer IN PLACE with dL/dlogits, so the lm_head
//             dgrad/wgrad GEMMs consume it directly
// z = logits / temperature.  Rows with label < 0 are ignored (logp = 0, zero gradient).
#include "common.cuh"

namespace b200 {

struct alignas(16) bf8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void online_merge(float& m, float& s, float& sz, float m2, float s2, float sz2) {
  const float nm = fmaxf(m, m2);
  const float a = (m == -INFINITY) ? 0.f : __expf(m - nm);
  const float b = (m2 == -INFINITY) ? 0.f : __expf(m2 - nm);
  s = s * a + s2 * b;
  sz = sz * a + sz2 * b;
  m = nm;
}

// VP (vocabulary parallel): `logits` holds the columns [label_offset, label_offset + V) of the full vocabulary.  Rows are
// skipped only when the GLOBAL label is negative; the outputs are this shard's partial results, combined across the
// tensor-parallel ranks by the caller: logp <- the label's scaled logit when it lies in this shard (else 0), lse_out <- the
// log-sum-exp over this shard, ent_out <- sum_i softmax_local(i) * z_i (the shard's mean scaled logit).
template <bool VP>
__global__ void __launch_bounds__(512)
logprob_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                   float* __restrict__ logp, float* __restrict__ lse_out, float* __restrict__ ent_out, int V,
                   long long ld, float inv_temp, long long label_offset) {
  __shared__ float sm[16], ss[16], sz_[16];
  const long long row = blockIdx.x;
  const long long glabel = labels[row];
  const long long label = VP ? glabel - label_offset : glabel;
  if (VP ? (glabel < 0) : (label < 0 || label >= V)) {
    if (threadIdx.x == 0) {
      logp[row] = 0.f;
      if (lse_out) lse_out[row] = 0.f;
      if (ent_out) ent_out[row] = 0.f;
    }
    return;
  }
  const __nv_bfloat16* r = logits + row * ld;
  float m = -INFINITY, s = 0.f, sz = 0.f;  // running max, sum exp(z-m), sum exp(z-m)*z
  const int nv = V / 8;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const bf8 p = reinterpret_cast<const bf8*>(r)[i];
    float z[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(p.v[j]);
      z[2 * j] = t.x * inv_temp;
      z[2 * j + 1] = t.y * inv_temp;
    }
    float cm = z[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, z[j]);
    if (cm > m) {
      const float a = __expf(m - cm);
      s *= a;
      sz *= a;
      m = cm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float e = __expf(z[j] - m);
      s += e;
      sz += e * z[j];
    }
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) {
    const float z = __bfloat162float(r[i]) * inv_temp;
    if (z > m) {
      const float a = __expf(m - z);
      s *= a;
      sz *= a;
      m = z;
    }
    const float e = __expf(z - m);
    s += e;
    sz += e * z;
  }
  // warp then block merge
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float z2 = __shfl_xor_sync(0xffffffffu, sz, o);
    online_merge(m, s, sz, m2, s2, z2);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) {
    sm[w] = m;
    ss[w] = s;
    sz_[w] = sz;
  }
  __syncthreads();
  if (w == 0) {
    m = lane < nw ? sm[lane] : -INFINITY;
    s = lane < nw ? ss[lane] : 0.f;
    sz = lane < nw ? sz_[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const float z2 = __shfl_xor_sync(0xffffffffu, sz, o);
      online_merge(m, s, sz, m2, s2, z2);
    }
    if (lane == 0) {
      const float lse = m + logf(s);
      if (VP) {
        logp[row] = (label >= 0 && label < V) ? __bfloat162float(r[label]) * inv_temp : 0.f;
        if (lse_out) lse_out[row] = lse;
        if (ent_out) ent_out[row] = sz / s;
      } else {
        const float zl = __bfloat162float(r[label]) * inv_temp;
        logp[row] = zl - lse;
        if (lse_out) lse_out[row] = lse;
        if (ent_out) ent_out[row] = lse - sz / s;
      }
    }
  }
}

// logits[row, v] <- g[row] * (1[v == label] - exp(z_v - lse)) * inv_temp      (bf16, in place)
// VP: `lse` is the GLOBAL log-sum-exp (over all shards) and the label is global; a label outside this shard just never matches.
template <bool VP>
__global__ void __launch_bounds__(512)
logprob_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                   const float* __restrict__ lse, const float* __restrict__ g, int V, long long ld, float inv_temp,
                   long long label_offset) {
  const long long row = blockIdx.x;
  const long long glabel = labels[row];
  const long long label = VP ? glabel - label_offset : glabel;
  __nv_bfloat16* r = logits + row * ld;
  const int nv = V / 8;
  const bool ignore = VP ? (glabel < 0) : (label < 0 || label >= V);
  const float gr = ignore ? 0.f : g[row];
  if (gr == 0.f) {
    bf8 z;
#pragma unroll
    for (int j = 0; j < 4; ++j) z.v[j] = __floats2bfloat162_rn(0.f, 0.f);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) reinterpret_cast<bf8*>(r)[i] = z;
    for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) r[i] = __float2bfloat16(0.f);
    return;
  }
  const float l = lse[row];
  const float gs = gr * inv_temp;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    bf8 p = reinterpret_cast<bf8*>(r)[i];
    const int base = i * 8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(p.v[j]);
      float d0 = -__expf(t.x * inv_temp - l);
      float d1 = -__expf(t.y * inv_temp - l);
      if (base + 2 * j == label) d0 += 1.f;
      if (base + 2 * j + 1 == label) d1 += 1.f;
      p.v[j] = __floats2bfloat162_rn(d0 * gs, d1 * gs);
    }
    reinterpret_cast<bf8*>(r)[i] = p;
  }
  for (int i = nv * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float d = -__expf(__bfloat162float(r[i]) * inv_temp - l);
    if (i == label) d += 1.f;
    r[i] = __float2bfloat16(d * gs);
  }
}

}  // namespace b200

using namespace b200;

// logits [T, V] bf16 (row stride ld, multiple of 8), labels [T] int64 (already shifted).
extern "C" int b200_logprob_fwd(const void* logits, const long long* labels, float* logp, float* lse, float* entropy,
                                int T, int V, long long ld, float temperature, void* stream) {
  if (T <= 0) return 0;
  if (ld % 8) return -1;
  logprob_fwd_kernel<false><<<T, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(logits), labels, logp, lse, entropy, V, ld, 1.f / temperature, 0);
  return static_cast<int>(cudaGetLastError());
}
// Vocabulary-parallel form: `logits` [T, V] are the columns [label_offset, label_offset + V) of the full vocabulary; see the
// kernel for what the three outputs hold.
extern "C" int b200_logprob_fwd_vp(const void* logits, const long long* labels, float* label_logit, float* lse_local,
                                   float* mean_logit_local, int T, int V, long long ld, float temperature,
                                   long long label_offset, void* stream) {
  if (T <= 0) return 0;
  if (ld % 8) return -1;
  logprob_fwd_kernel<true><<<T, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(logits), labels, label_logit, lse_local, mean_logit_local, V, ld, 1.f / temperature,
      label_offset);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int b200_logprob_bwd(void* logits, const long long* labels, const float* lse, const float* g, int T, int V,
                                long long ld, float temperature, void* stream) {
  if (T <= 0) return 0;
  if (ld % 8) return -1;
  logprob_bwd_kernel<false><<<T, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(logits), labels, lse, g, V, ld, 1.f / temperature, 0);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int b200_logprob_bwd_vp(void* logits, const long long* labels, const float* lse_global, const float* g, int T, int V,
                                   long long ld, float temperature, long long label_offset, void* stream) {
  if (T <= 0) return 0;
  if (ld % 8) return -1;
  logprob_bwd_kernel<true><<<T, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(logits), labels, lse_global, g, V, ld, 1.f / temperature, label_offset);
  return static_cast<int>(cudaGetLastError());
}
