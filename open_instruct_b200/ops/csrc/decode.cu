// Rollout-engine kernels: paged KV cache writes, paged decode attention (GQA, split-KV) and
// token sampling with log-probs of the processed distribution.
//
// KV cache layout per layer: [num_blocks, Hkv, BLOCK, Dh] bf16 for K and for V (BLOCK = 64 tokens),
// so one (block, kv head) pair is a contiguous 16 KB tile.  A sequence owns a list of block ids
// (its row of the block table); several sequences may point at the same prompt blocks.
//
// Decode attention is bandwidth work (every cached key and value is read once per step): one CTA
// per (sequence, kv head, split) streams its share of the blocks, all G = Hq/Hkv query heads of
// the group are served from the same K/V reads, partial (max, sum, out) triples are merged by a
// second kernel when the sequence was split.
#include "common.cuh"
#include <atomic>
#include <cstdlib>

namespace b200 {

constexpr int KV_BLOCK = 64;
constexpr int DEC_DH = 128;
constexpr int MAX_G = 8;

// ------------------------------------------------------------------ KV cache write
// qkv [T, (Hq+2Hkv)*Dh] (post-RoPE) -> cache at slot_mapping[t] = block_id * BLOCK + offset (-1: skip)
// `slots` has T entries; entry t takes its K/V from qkv row (t % T_src), so one launch can place the
// same tokens at several destinations (samples of one prompt that own private tail blocks).
__global__ void kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                                __nv_bfloat16* __restrict__ vc, const long long* __restrict__ slots, int T, int T_src, int Hq,
                                int Hkv) {
  const long long row_stride = static_cast<long long>(Hq + 2 * Hkv) * DEC_DH;
  const int vec_per_tok = Hkv * DEC_DH / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < static_cast<long long>(T) * vec_per_tok;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vec_per_tok;
    const int v = static_cast<int>(i % vec_per_tok);
    const long long slot = slots[t];
    if (slot < 0) continue;
    const int h = v / (DEC_DH / 8), d8 = v % (DEC_DH / 8);
    const long long blk = slot / KV_BLOCK, off = slot % KV_BLOCK;
    const long long dst = ((blk * Hkv + h) * KV_BLOCK + off) * DEC_DH + d8 * 8;
    const __nv_bfloat16* src = qkv + (t % T_src) * row_stride + static_cast<long long>(Hq + h) * DEC_DH + d8 * 8;
    *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(src);
    *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(src + static_cast<long long>(Hkv) * DEC_DH);
  }
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&f)[8]) {
  f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
  f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
  f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
  f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
}

// Decode step: rotary embedding of the new token's q and k heads (cos/sin from the table) AND the write of its rotated K
// and its V into the paged cache, in one pass over the fused qkv row (one launch instead of two per layer).
// One thread handles 8 (lo, hi) pairs of one head; v heads are copied.  slots[t] < 0 skips the cache write.
__global__ void rope_kv_decode_kernel(__nv_bfloat16* __restrict__ qkv, const float2* __restrict__ tab, __nv_bfloat16* __restrict__ kc,
                                      __nv_bfloat16* __restrict__ vc, const long long* __restrict__ slots, long long T, int Hq,
                                      int Hkv) {
  griddep_launch_dependents();
  griddep_wait();
  constexpr int half = DEC_DH / 2, nchunk = half / 8;
  const int heads = Hq + 2 * Hkv;
  const long long row_stride = static_cast<long long>(heads) * DEC_DH;
  const long long total = T * heads * nchunk;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % nchunk);
    const long long th = idx / nchunk;
    const int hd = static_cast<int>(th % heads);
    const long long t = th / heads;
    __nv_bfloat16* base = qkv + t * row_stride + static_cast<long long>(hd) * DEC_DH + c * 8;
    uint4 ulo = *reinterpret_cast<const uint4*>(base), uhi = *reinterpret_cast<const uint4*>(base + half);
    if (hd < Hq + Hkv) {
      float lo[8], hi[8];
      unpack_bf16x8(ulo, lo);
      unpack_bf16x8(uhi, hi);
      const float4* tv = reinterpret_cast<const float4*>(tab + t * half + c * 8);
      float ol[8], oh[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 cs = tv[j];  // (cos, sin) of pairs 2j and 2j + 1
        ol[2 * j] = lo[2 * j] * cs.x - hi[2 * j] * cs.y;
        oh[2 * j] = hi[2 * j] * cs.x + lo[2 * j] * cs.y;
        ol[2 * j + 1] = lo[2 * j + 1] * cs.z - hi[2 * j + 1] * cs.w;
        oh[2 * j + 1] = hi[2 * j + 1] * cs.z + lo[2 * j + 1] * cs.w;
      }
      ulo = make_uint4(pack_bf16x2(ol[0], ol[1]), pack_bf16x2(ol[2], ol[3]), pack_bf16x2(ol[4], ol[5]), pack_bf16x2(ol[6], ol[7]));
      uhi = make_uint4(pack_bf16x2(oh[0], oh[1]), pack_bf16x2(oh[2], oh[3]), pack_bf16x2(oh[4], oh[5]), pack_bf16x2(oh[6], oh[7]));
      *reinterpret_cast<uint4*>(base) = ulo;
      *reinterpret_cast<uint4*>(base + half) = uhi;
      if (hd < Hq) continue;
    }
    const long long slot = slots[t];
    if (slot < 0) continue;
    const bool is_v = hd >= Hq + Hkv;
    const int h = hd - Hq - (is_v ? Hkv : 0);
    const long long blk = slot / KV_BLOCK, off = slot % KV_BLOCK;
    __nv_bfloat16* dst = (is_v ? vc : kc) + ((blk * Hkv + h) * KV_BLOCK + off) * DEC_DH + c * 8;
    *reinterpret_cast<uint4*>(dst) = ulo;
    *reinterpret_cast<uint4*>(dst + half) = uhi;
  }
}

// ------------------------------------------------------------------ paged decode attention
// q rows come from qkv [B, (Hq+2Hkv)*Dh]; context length of sequence b is ctx[b] (keys 0..ctx-1,
// the new token's K/V already written).  grid = (B, Hkv, splits), 128 threads.
template <int G>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table, int max_blocks,
                    const int* __restrict__ ctx, int Hq, int Hkv, float scale, int splits,
                    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml) {
  __shared__ float sq[G][DEC_DH];
  __shared__ float sp[G][KV_BLOCK];
  __shared__ float red[G][4];
  const int b = blockIdx.x, kvh = blockIdx.y, sp_i = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = ctx[b];
  const int nblk = (L + KV_BLOCK - 1) / KV_BLOCK;
  const int per = (nblk + splits - 1) / splits;
  const int blk0 = sp_i * per, blk1 = min(nblk, blk0 + per);
  const long long row_stride = static_cast<long long>(Hq + 2 * Hkv) * DEC_DH;
  for (int i = tid; i < G * DEC_DH; i += 128) {
    const int g = i / DEC_DH, d = i % DEC_DH;
    sq[g][d] = __bfloat162float(qkv[b * row_stride + static_cast<long long>(kvh * G + g) * DEC_DH + d]) * scale;
  }
  __syncthreads();
  float m[G], l[G], acc[G];
#pragma unroll
  for (int g = 0; g < G; ++g) { m[g] = -INFINITY; l[g] = 0.f; acc[g] = 0.f; }
  // thread -> (key within block, half of the group's heads) for scores; thread -> dim for PV
  const int key = tid & 63, gh = tid >> 6;  // gh in {0,1}
  constexpr int GH = (G + 1) / 2;
  for (int bi = blk0; bi < blk1; ++bi) {
    const long long blk = block_table[static_cast<long long>(b) * max_blocks + bi];
    const __nv_bfloat16* kt = kc + ((blk * Hkv + kvh) * KV_BLOCK) * DEC_DH;
    const __nv_bfloat16* vt = vc + ((blk * Hkv + kvh) * KV_BLOCK) * DEC_DH;
    const int kpos = bi * KV_BLOCK + key;
    float s[GH];
#pragma unroll
    for (int j = 0; j < GH; ++j) s[j] = 0.f;
    if (kpos < L) {
      const uint4* kr = reinterpret_cast<const uint4*>(kt + key * DEC_DH);
#pragma unroll 4
      for (int c = 0; c < DEC_DH / 8; ++c) {
        const uint4 u = kr[c];
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
        float kf[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p2[e]); kf[2 * e] = f.x; kf[2 * e + 1] = f.y; }
#pragma unroll
        for (int j = 0; j < GH; ++j) {
          const int g = gh * GH + j;
          if (g < G) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s[j] += kf[e] * sq[g][c * 8 + e];
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < GH; ++j) {
      const int g = gh * GH + j;
      if (g < G) sp[g][key] = kpos < L ? s[j] : -INFINITY;
    }
    __syncthreads();
    // block max per head (every thread computes all heads' maxima from shared memory via warp 0..3 partials)
    float bm[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = fmaxf(sp[g][lane], sp[g][lane + 32]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      bm[g] = v;
    }
    float alpha[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float mn = fmaxf(m[g], bm[g]);
      alpha[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mn);
      m[g] = mn;
    }
    __syncthreads();
    // probabilities in place + block sums
#pragma unroll
    for (int j = 0; j < GH; ++j) {
      const int g = gh * GH + j;
      if (g < G) {
        const float sv = sp[g][key];
        sp[g][key] = (sv == -INFINITY) ? 0.f : __expf(sv - m[g]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float v = sp[g][lane] + sp[g][lane + 32];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      l[g] = l[g] * alpha[g] + v;
      acc[g] *= alpha[g];
    }
    // PV: thread tid owns output dim tid for every head of the group
    const int kmax = min(KV_BLOCK, L - bi * KV_BLOCK);
    for (int k = 0; k < kmax; ++k) {
      const float vv = __bfloat162float(vt[k * DEC_DH + tid]);
#pragma unroll
      for (int g = 0; g < G; ++g) acc[g] += sp[g][k] * vv;
    }
    __syncthreads();
  }
  (void)warp; (void)red;
  if (splits == 1) {
#pragma unroll
    for (int g = 0; g < G; ++g)
      out[(static_cast<long long>(b) * Hq + kvh * G + g) * DEC_DH + tid] = __float2bfloat16(l[g] > 0.f ? acc[g] / l[g] : 0.f);
  } else {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const long long idx = (static_cast<long long>(b) * Hq + kvh * G + g) * splits + sp_i;
      part_o[idx * DEC_DH + tid] = acc[g];
      if (tid == 0) { part_ml[idx * 2] = m[g]; part_ml[idx * 2 + 1] = l[g]; }
    }
  }
}


// ------------------------------------------------------------------ paged decode attention, streaming form
// Same contract as paged_decode_kernel.  Layout of the work: a half-warp reads one 256-byte K (or V) row per load
// instruction (lane -> 8 of the 128 dims), so every request is a full contiguous row; a thread owns KPT consecutive keys
// of each 8*KPT-key slice (warp w, half-warp h -> keys (2w+h)*KPT ...).  The K rows of the NEXT slice and the V rows of
// this one are requested before this slice's scores are computed, so 2*KPT 16-byte loads per thread are in flight
// while the arithmetic runs.  Every warp keeps its own running (max, sum, output) over the keys it sees: the main loop
// has no block-wide barrier; the four warps are merged once at the end, exactly like split-KV partials.
//
// Scores: each thread forms partial dot products over its 8 dims for NK keys x GP heads (NK * GP = 16) and the 16
// values are summed over the 16 lanes by recursive halving (15 shuffles): lane i ends up with the complete score of
// (key i / GP, head i % GP).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

template <int N>
__device__ __forceinline__ void halve_reduce(float (&v)[16], int l16) {
  if constexpr (N >= 2) {
    constexpr int H = N / 2;
    const bool upper = (l16 & H) != 0;  // mask H: 8, 4, 2, 1 for N = 16, 8, 4, 2
#pragma unroll
    for (int j = 0; j < H; ++j) {
      const float send = upper ? v[j] : v[j + H];
      const float keep = upper ? v[j + H] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, H);
    }
    halve_reduce<H>(v, l16);
  }
}

template <int G, int KPT, int MINB>
__global__ void __launch_bounds__(128, MINB)
paged_decode_stream_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ kc,
                           const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ ctx, int Hq, int Hkv, float scale, int splits,
                           __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml) {
  griddep_launch_dependents();  // the o_proj GEMM that follows may bring its first weight tiles in during this kernel's tail
  griddep_wait();               // launched with programmatic serialization: q and the new K/V rows are the predecessor's output
  constexpr int GP = G <= 2 ? 2 : (G <= 4 ? 4 : 8);  // heads padded to a power of two
  constexpr int NK = 16 / GP;                         // keys per reduction batch
  static_assert(KPT % NK == 0, "keys per thread must be whole reduction batches");
  constexpr int NB = KPT / NK;
  constexpr int KI = 8 * KPT;                         // keys per block iteration (all four warps)
  static_assert(KV_BLOCK % KI == 0, "an iteration must not straddle pages");
  constexpr int IPP = KV_BLOCK / KI;
  __shared__ __align__(16) float sp[4][2 * KPT][GP];
  __shared__ __align__(16) float sal[4][GP];
  __shared__ __align__(16) float so[4][G][DEC_DH];
  __shared__ float sml[4][G][2];
  const int b = blockIdx.x, kvh = blockIdx.y, sp_i = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, l16 = lane & 15, hw = lane >> 4;
  const int L = ctx[b];
  const int nblk = (L + KV_BLOCK - 1) / KV_BLOCK;
  const int per = (nblk + splits - 1) / splits;
  const int blk0 = sp_i * per, blk1 = min(nblk, blk0 + per);
  const int it0 = blk0 * IPP, it1 = blk1 * IPP;
  const long long row_stride = static_cast<long long>(Hq + 2 * Hkv) * DEC_DH;

  float q[G][8];
  {
    const __nv_bfloat16* qrow = qkv + b * row_stride + static_cast<long long>(kvh * G) * DEC_DH + l16 * 8;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const uint4 u = *reinterpret_cast<const uint4*>(qrow + g * DEC_DH);
      unpack_bf16x8(u, q[g]);
#pragma unroll
      for (int e = 0; e < 8; ++e) q[g][e] *= scale;
    }
  }
  float acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  float m_l = -INFINITY, l_l = 0.f;  // running max / partial sum of head (lane % GP) over this warp's keys
  const int kbase = (warp * 2 + hw) * KPT;
  const int* bt_row = block_table + static_cast<long long>(b) * max_blocks;

  uint4 k_cur[KPT], k_nxt[KPT], v_cur[KPT];
  auto load_slice = [&](int it, const __nv_bfloat16* base, uint4 (&r)[KPT]) {
    const long long blk = bt_row[it / IPP];
    const __nv_bfloat16* p = base + ((blk * Hkv + kvh) * KV_BLOCK + (it % IPP) * KI + kbase) * DEC_DH + l16 * 8;
    const int k0 = it * KI + kbase;
#pragma unroll
    for (int j = 0; j < KPT; ++j) r[j] = (k0 + j < L) ? ld_stream16(p + j * DEC_DH) : make_uint4(0u, 0u, 0u, 0u);
  };
  if (it0 < it1) load_slice(it0, kc, k_cur);
  for (int it = it0; it < it1; ++it) {
    load_slice(it, vc, v_cur);
    if (it + 1 < it1) load_slice(it + 1, kc, k_nxt);
    const int k0 = it * KI + kbase;
    float sc[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float v[16];
#pragma unroll
      for (int kk = 0; kk < NK; ++kk) {
        float kf[8];
        unpack_bf16x8(k_cur[nb * NK + kk], kf);
#pragma unroll
        for (int g = 0; g < GP; ++g) {
          float d = 0.f;
          if (g < G) {
#pragma unroll
            for (int e = 0; e < 8; ++e) d = fmaf(kf[e], q[g < G ? g : 0][e], d);
          }
          v[kk * GP + g] = d;
        }
      }
      halve_reduce<16>(v, l16);
      const int kpos = k0 + nb * NK + l16 / GP;
      sc[nb] = (kpos < L && (l16 % GP) < G) ? v[0] : -INFINITY;
    }
    float tmax = sc[0];
#pragma unroll
    for (int nb = 1; nb < NB; ++nb) tmax = fmaxf(tmax, sc[nb]);
#pragma unroll
    for (int o = GP; o < 32; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    const float m_new = fmaxf(m_l, tmax);
    const float alpha = (m_l == -INFINITY) ? 0.f : __expf(m_l - m_new);
    float psum = 0.f;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const float pv = (sc[nb] == -INFINITY) ? 0.f : __expf(sc[nb] - m_new);
      psum += pv;
      sp[warp][hw * KPT + nb * NK + l16 / GP][l16 % GP] = pv;
    }
    l_l = l_l * alpha + psum;
    m_l = m_new;
    if (lane < GP) sal[warp][lane] = alpha;
    __syncwarp();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float a = sal[warp][g];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= a;
    }
#pragma unroll
    for (int j = 0; j < KPT; ++j) {
      float vf[8];
      unpack_bf16x8(v_cur[j], vf);
      float pj[GP];
      if constexpr (GP == 2) {
        const float2 t = *reinterpret_cast<const float2*>(&sp[warp][hw * KPT + j][0]);
        pj[0] = t.x; pj[1] = t.y;
      } else {
#pragma unroll
        for (int c = 0; c < GP / 4; ++c) {
          const float4 t = *reinterpret_cast<const float4*>(&sp[warp][hw * KPT + j][4 * c]);
          pj[4 * c] = t.x; pj[4 * c + 1] = t.y; pj[4 * c + 2] = t.z; pj[4 * c + 3] = t.w;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pj[g], vf[e], acc[g][e]);
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < KPT; ++j) k_cur[j] = k_nxt[j];
  }
  // merge: the two half-warps, then the four warps (each with its own running maximum)
#pragma unroll
  for (int o = GP; o < 32; o <<= 1) l_l += __shfl_xor_sync(0xffffffffu, l_l, o);
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], 16);
  if (hw == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      *reinterpret_cast<float4*>(&so[warp][g][l16 * 8]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
      *reinterpret_cast<float4*>(&so[warp][g][l16 * 8 + 4]) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    }
  }
  if (lane < GP && lane < G) { sml[warp][lane][0] = m_l; sml[warp][lane][1] = l_l; }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sml[w][g][0]);
    float o = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sml[w][g][0];
      const float wt = (mw == -INFINITY) ? 0.f : __expf(mw - M);
      o += wt * so[w][g][tid];
      lsum += wt * sml[w][g][1];
    }
    if (splits == 1) {
      out[(static_cast<long long>(b) * Hq + kvh * G + g) * DEC_DH + tid] = __float2bfloat16(lsum > 0.f ? o / lsum : 0.f);
    } else {
      const long long idx = (static_cast<long long>(b) * Hq + kvh * G + g) * splits + sp_i;
      part_o[idx * DEC_DH + tid] = o;
      if (tid == 0) { part_ml[idx * 2] = M; part_ml[idx * 2 + 1] = lsum; }
    }
  }
}

__global__ void __launch_bounds__(128)
decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                      __nv_bfloat16* __restrict__ out) {
  const long long bh = blockIdx.x;
  const int d = threadIdx.x;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_ml[(bh * splits + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(bh * splits + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - mx);
    l += part_ml[(bh * splits + s) * 2 + 1] * w;
    o += part_o[(bh * splits + s) * DEC_DH + d] * w;
  }
  out[bh * DEC_DH + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
}

// ------------------------------------------------------------------ sampling
// Philox4x32-10 counter RNG: (seed, row counter, token index) -> uniform in (0, 1).
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0];
  const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
  const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
  const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
  c[1] = static_cast<uint32_t>(p1);
  c[3] = static_cast<uint32_t>(p0);
  c[0] = n0;
  c[2] = n2;
}
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t ctr_hi, uint32_t ctr_lo, uint32_t idx) {
  uint32_t c[4] = {idx, ctr_lo, ctr_hi, 0u};
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return (static_cast<float>(c[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax argmax_merge(ArgMax a, ArgMax b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

// One CTA per row.  temperature == 0 -> greedy.  top_p in (0, 1]: nucleus found by bisection on the
// probability threshold (each iteration one pass over the row, L2 resident).
// Outputs: token id, log-prob of that token under the processed (temperature + top-p renormalised)
// distribution.
__global__ void __launch_bounds__(1024)
sample_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const long long* __restrict__ seeds, const int* __restrict__ counters,
              long long* __restrict__ tokens, float* __restrict__ logprobs) {
  griddep_launch_dependents();
  griddep_wait();
  __shared__ float sred[32];
  __shared__ ArgMax samax[32];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const __nv_bfloat16* r = logits + static_cast<long long>(row) * ld;
  const float temp = temperature[row];
  const bool greedy = temp <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  auto block_max = [&](float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) sred[warp] = v;
    __syncthreads();
    float x = lane < nw ? sred[lane] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
  };
  auto block_sum = [&](float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sred[warp] = v;
    __syncthreads();
    float x = lane < nw ? sred[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
  };
  float mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, __bfloat162float(r[i]) * inv_t);
  mx = block_max(mx);
  float sum = 0.f;
  for (int i = tid; i < V; i += blockDim.x) sum += __expf(__bfloat162float(r[i]) * inv_t - mx);
  sum = block_sum(sum);
  // nucleus threshold (on exp(z - mx), i.e. unnormalised probabilities)
  float thr = 0.f, kept = sum;
  const float tp = top_p ? top_p[row] : 1.f;
  if (!greedy && tp < 1.f) {
    float lo = 0.f, hi = 1.f;  // exp(z - mx) lies in (0, 1]
    const float target = tp * sum;
    for (int it = 0; it < 24; ++it) {
      const float mid = 0.5f * (lo + hi);
      float s = 0.f;
      for (int i = tid; i < V; i += blockDim.x) {
        const float e = __expf(__bfloat162float(r[i]) * inv_t - mx);
        if (e >= mid) s += e;
      }
      s = block_sum(s);
      if (s >= target) lo = mid; else hi = mid;  // keep the largest threshold whose mass still reaches top_p
    }
    thr = lo;
    float s = 0.f;
    for (int i = tid; i < V; i += blockDim.x) {
      const float e = __expf(__bfloat162float(r[i]) * inv_t - mx);
      if (e >= thr) s += e;
    }
    kept = block_sum(s);
  }
  // Gumbel-max over the kept set (plain argmax when greedy)
  const uint64_t seed = static_cast<uint64_t>(seeds ? seeds[row] : 0);
  const uint32_t ctr = counters ? static_cast<uint32_t>(counters[row]) : 0u;
  ArgMax best = {-INFINITY, 0x7fffffff};
  for (int i = tid; i < V; i += blockDim.x) {
    const float z = __bfloat162float(r[i]) * inv_t - mx;
    float score;
    if (greedy) {
      score = z;
    } else {
      if (__expf(z) < thr) continue;
      const float u = philox_uniform(seed, 0u, ctr, static_cast<uint32_t>(i));
      score = z - __logf(-__logf(u));
    }
    best = argmax_merge(best, ArgMax{score, i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = argmax_merge(best, other);
  }
  __syncthreads();
  if (lane == 0) samax[warp] = best;
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? samax[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = argmax_merge(best, other);
    }
    if (lane == 0) {
      const int tok = best.i < V ? best.i : 0;
      tokens[row] = tok;
      const float z = __bfloat162float(r[tok]) * inv_t - mx;
      logprobs[row] = z - __logf(greedy ? sum : kept);
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_kv_write(const void* qkv, void* k_cache, void* v_cache, const long long* slots, int T, int T_src, int Hq,
                             int Hkv, int Dh, void* stream) {
  if (T <= 0 || T_src <= 0) return 0;
  if (Dh != DEC_DH) return -1;
  const long long work = static_cast<long long>(T) * Hkv * DEC_DH / 8;
  int grid = static_cast<int>((work + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  kv_write_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<__nv_bfloat16*>(k_cache),
      reinterpret_cast<__nv_bfloat16*>(v_cache), slots, T, T_src, Hq, Hkv);
  return static_cast<int>(cudaGetLastError());
}

static std::atomic<int> g_decode_variant{[] { const char* e = getenv("B200_DECODE_ATTN"); return e ? atoi(e) : 0; }()};
// which decode-attention kernel b200_paged_decode launches (see there)
extern "C" int b200_paged_decode_variant(int v) {
  g_decode_variant.store(v);
  return 0;
}

// qkv [T, (Hq + 2 Hkv) * 128] in place; table [T, 64] float2 (cos, sin); slots [T] cache positions of the tokens (-1: skip)
extern "C" int b200_rope_kv_decode(void* qkv, const void* table, void* k_cache, void* v_cache, const long long* slots, int T, int Hq,
                                   int Hkv, int Dh, void* stream) {
  if (T <= 0) return 0;
  if (Dh != DEC_DH) return -1;
  const long long total = static_cast<long long>(T) * (Hq + 2 * Hkv) * (DEC_DH / 16);
  long long grid = (total + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  cudaError_t le = launch_pdl(rope_kv_decode_kernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                              reinterpret_cast<__nv_bfloat16*>(qkv), reinterpret_cast<const float2*>(table),
                              reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache), slots,
                              static_cast<long long>(T), Hq, Hkv);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}

// scratch (only read when splits > 1): part_o [B*Hq*splits*128] floats, part_ml [B*Hq*splits*2] floats
extern "C" int b200_paged_decode(const void* qkv, const void* k_cache, const void* v_cache, const int* block_table,
                                 int max_blocks, const int* ctx, int B, int Hq, int Hkv, int Dh, float scale, int splits,
                                 void* out, float* part_o, float* part_ml, void* stream) {
  if (B <= 0) return 0;
  if (Dh != DEC_DH || Hq % Hkv) return -1;
  const int G = Hq / Hkv;
  if (splits < 1) splits = 1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(B, Hkv, splits);
  // variant: 0 = streaming kernel (default; 4 keys per thread and iteration at group size 4: 97 us against 104 us with 8 at
  // 256 sequences of 256-512 tokens), 1 = the block-synchronous kernel (213 us there), 2 = streaming with 8 keys per thread
  const int variant = g_decode_variant.load(std::memory_order_relaxed);
#define B200_DECS(GV, KPT, MINB)                                                                                       \
  launch_pdl(paged_decode_stream_kernel<GV, KPT, MINB>, grid, dim3(128), 0, st,                                        \
             reinterpret_cast<const __nv_bfloat16*>(qkv), reinterpret_cast<const __nv_bfloat16*>(k_cache),             \
             reinterpret_cast<const __nv_bfloat16*>(v_cache), block_table, max_blocks, ctx, Hq, Hkv, scale, splits,    \
             reinterpret_cast<__nv_bfloat16*>(out), part_o, part_ml)
  bool launched = variant != 1;
  if (variant != 1) {
    switch (G) {
      case 1: B200_DECS(1, 8, 2); break;
      case 2: B200_DECS(2, 8, 2); break;
      case 4: if (variant == 2) B200_DECS(4, 8, 2); else B200_DECS(4, 4, 3); break;
      case 7: B200_DECS(7, 4, 2); break;
      case 8: B200_DECS(8, 4, 2); break;
      default: launched = false;
    }
  }
#undef B200_DECS
#define B200_DEC(GV)                                                                                                   \
  paged_decode_kernel<GV><<<grid, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(qkv),                           \
                                                reinterpret_cast<const __nv_bfloat16*>(k_cache),                        \
                                                reinterpret_cast<const __nv_bfloat16*>(v_cache), block_table, max_blocks, \
                                                ctx, Hq, Hkv, scale, splits, reinterpret_cast<__nv_bfloat16*>(out), part_o, \
                                                part_ml)
  if (!launched) {
    switch (G) {
      case 1: B200_DEC(1); break;
      case 2: B200_DEC(2); break;
      case 4: B200_DEC(4); break;
      case 7: B200_DEC(7); break;
      case 8: B200_DEC(8); break;
      default: return -2;
    }
  }
#undef B200_DEC
  if (splits > 1)
    decode_combine_kernel<<<B * Hq, 128, 0, st>>>(part_o, part_ml, splits, reinterpret_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_sample(const void* logits, long long ld, int B, int V, const float* temperature, const float* top_p,
                           const long long* seeds, const int* counters, long long* tokens, float* logprobs, void* stream) {
  if (B <= 0) return 0;
  cudaError_t le = launch_pdl(sample_kernel, dim3(B), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream),
                              reinterpret_cast<const __nv_bfloat16*>(logits), ld, V, temperature, top_p, seeds, counters, tokens, logprobs);
  return static_cast<int>(le != cudaSuccess ? le : cudaGetLastError());
}
