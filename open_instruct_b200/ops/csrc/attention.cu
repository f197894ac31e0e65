// Padding-free (varlen) causal attention for packed sequences, GQA, head_dim 128, on tcgen05.
//
// Layout: fused qkv [T, (Hq + 2*Hkv) * 128] bf16 (q heads | k heads | v heads per token, RoPE
// already applied), cu_seqlens [B+1] int32 document boundaries, out [T, Hq*128] bf16,
// lse [Hq, T] fp32 (natural log of the softmax denominator of scale*QK^T).
//
// Forward: one CTA per (128-query tile, q head).  Warp 0 streams K/V tiles with TMA, warp 1
// issues S = Q K^T (double-buffered in TMEM) and O += P V (accumulated in TMEM), warps 2-5 own one
// query row per thread: the score row is read from TMEM once into registers, the softmax maximum
// follows the row maximum lazily (O is rescaled in TMEM only when it moved by more than 2^8), P is
// written to swizzled shared memory as bf16 while the previous P V still runs.
//
// Backward: one CTA per (128-key tile, kv head); it walks every query tile at or after its key
// tile for each q head of the GQA group.  Scores are computed transposed (S^T = K Q^T) so each
// thread owns one key row; dK and dV accumulate in TMEM across the whole walk, dQ tiles are
// reduced into an fp32 scratch with vector red.global and converted once at the end.
#include "common.cuh"

namespace b200 {

constexpr int DH = 128;
constexpr int TQ = 128;   // query tile
constexpr int TK = 128;   // key tile
constexpr int SUB = 128 * 64 * 2;  // bytes of one [128 x 64] bf16 swizzled sub-tile (16 KB)
constexpr int TILE = 2 * SUB;      // [128 x 128] bf16 tile (32 KB)
constexpr int ATT_THREADS = 192;
constexpr int BWD_THREADS = 320;  // TMA warp, MMA warp, 8 compute warps (two per TMEM lane quarter, 64 columns each)
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ bool find_tile(const int* __restrict__ cu, int B, int slot, int& start, int& end,
                                          int& tile, int& ntiles) {
  for (int b = 0; b < B; ++b) {
    const int s = cu[b], e = cu[b + 1];
    const int nt = (e - s + 127) / 128;
    if (slot < nt) {
      start = s;
      end = e;
      tile = slot;
      ntiles = nt;
      return true;
    }
    slot -= nt;
  }
  return false;
}

// offset (bytes) of the 16-byte chunk holding elements [col, col+8) of row `r` inside a
// [128 x 128] bf16 tile stored as two 128B-swizzled [128 x 64] sub-tiles
__device__ __forceinline__ uint32_t swz_off(int r, int col) {
  const int sub = col >> 6;
  const int chunk = (col & 63) >> 3;
  return sub * SUB + r * 128 + ((chunk ^ (r & 7)) << 4);
}

__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}

// K-major [128 x 128] tile operand: k-step `k` (16 elements) lives in sub-tile k/4
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int k) {
  return umma_desc_sw128(tile_addr + (k >> 2) * SUB + (k & 3) * 32, 16, 1024);
}
// MN-major view of a [128 rows(K) x 128 cols(MN)] tile: 16 K-rows per step, 64-wide MN blocks SUB apart
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int k) {
  return umma_desc_sw128(tile_addr + k * 2048, SUB, 1024);
}

// ===================================================================== forward
struct FwdSmem {
  uint8_t q[TILE];
  uint8_t k[2][TILE];
  uint8_t v[2][TILE];
  uint8_t p[TILE];
  uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full, o_full;
  uint32_t tmem_ptr;
  int abort_flag;
};

__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const int* __restrict__ cu, int B, int Hq, int Hkv,
                __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int T, float scale,
                int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int doc_start, doc_end, tile, ntiles;
  if (!find_tile(cu, B, blockIdx.x, doc_start, doc_end, tile, ntiles)) return;
  tile = ntiles - 1 - tile;  // longest rows first
  const int h = blockIdx.y;
  const int kvh = h / (Hq / Hkv);
  const int q0 = doc_start + tile * TQ;
  const int n_kv = tile + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.v_full[i], 1);
      mbar_init(&sm.k_empty[i], 1);
      mbar_init(&sm.v_empty[i], 1);
      mbar_init(&sm.s_full[i], 1);
    }
    mbar_init(&sm.p_full, 128);
    mbar_init(&sm.o_full, 1);
    sm.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_ptr;
  const uint32_t T_S0 = tmem, T_O = tmem + 256;  // S buffers at columns 0 and 128

  const int qcol = h * DH, kcol = (Hq + kvh) * DH, vcol = (Hq + Hkv + kvh) * DH;

  if (warp == 0) {
    if (elect_one()) {
      prefetch_tensormap(&tm_qkv);
      mbar_expect_tx(&sm.q_full, TILE);
      tma_load_2d(sm.q, &tm_qkv, &sm.q_full, qcol, q0);
      tma_load_2d(sm.q + SUB, &tm_qkv, &sm.q_full, qcol + 64, q0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int k0 = doc_start + j * TK;
        if (!mbar_wait(&sm.k_empty[s], ph ^ 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_EMPTY); break; }
        mbar_expect_tx(&sm.k_full[s], TILE);
        tma_load_2d(sm.k[s], &tm_qkv, &sm.k_full[s], kcol, k0);
        tma_load_2d(sm.k[s] + SUB, &tm_qkv, &sm.k_full[s], kcol + 64, k0);
        if (!mbar_wait(&sm.v_empty[s], ph ^ 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_EMPTY); break; }
        mbar_expect_tx(&sm.v_full[s], TILE);
        tma_load_2d(sm.v[s], &tm_qkv, &sm.v_full[s], vcol, k0);
        tma_load_2d(sm.v[s] + SUB, &tm_qkv, &sm.v_full[s], vcol + 64, k0);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128, false, true);
      const uint32_t q_addr = smem_u32(sm.q), p_addr = smem_u32(sm.p);
      bool ok = mbar_wait(&sm.q_full, 0, abort_flag);
      if (!ok) atomicCAS(status, 0, ST_TIMEOUT_FULL);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&sm.k_full[s], (j >> 1) & 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_FULL); return false; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sm.k[s]);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(T_S0 + s * 128, desc_kmajor(q_addr, k), desc_kmajor(k_addr, k), idesc_s, k != 0);
        umma_commit(&sm.k_empty[s]);
        umma_commit(&sm.s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j & 1;
        if (!mbar_wait(&sm.p_full, j & 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_TMEM_EMPTY); break; }
        if (!mbar_wait(&sm.v_full[s], (j >> 1) & 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_FULL); break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sm.v[s]);
#pragma unroll
        // O accumulates in TMEM over all key tiles; the softmax warps rescale it in place when a row maximum moves
        for (int k = 0; k < 8; ++k) umma_ss(T_O, desc_kmajor(p_addr, k), desc_mnmajor(v_addr, k), idesc_o, (j | k) != 0);
        umma_commit(&sm.v_empty[s]);
        umma_commit(&sm.o_full);
      }
    }
  } else {
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;          // query row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(lane_grp * 32) << 16;
    const float c = scale * LOG2E;
    // `m` is the maximum the exponentials are taken against.  It follows the true row maximum lazily: it moves only
    // when the row maximum has grown by more than 2^8 since, so the running output in TMEM is rescaled rarely and the
    // weights stay below 2^8 (exact in the end: O and l use the same m).
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      ok = warp_wait(&sm.s_full[s], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (j == n_kv - 1);
      const uint32_t ts = T_S0 + s * 128 + lane_off;
      uint32_t sv[4][32];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) tmem_ld32(ts + cc * 32, sv[cc]);
      tmem_ld_wait();
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(sv[cc][i]);
          if (diag && cc * 32 + i > r) {
            v = -INFINITY;  // causal mask: contributes exp2(-inf) = 0 below
            sv[cc][i] = __float_as_uint(v);
          }
          mx4[i & 3] = fmaxf(mx4[i & 3], v);
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float alpha = 1.f;
      const bool grow = (mx - m) * c > 8.f;
      if (grow) {
        alpha = ex2_approx((m - mx) * c);
        m = mx;
        l *= alpha;
      }
      const bool rescale = j > 0 && __any_sync(0xffffffffu, grow);
      const float mc = m * c;
      uint32_t pk[64];
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(sv[cc][i]), c, -mc));
          const float p1 = ex2_approx(fmaf(__uint_as_float(sv[cc][i + 1]), c, -mc));
          rs4[(i >> 1) & 3] += p0 + p1;
          pk[cc * 16 + (i >> 1)] = pack_bf16x2(p0, p1);
        }
      }
      l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      // the P buffer and the O accumulator are free once P V of the previous tile has completed
      if (j > 0) {
        ok = warp_wait(&sm.o_full, (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
      }
      if (rescale) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t t[32];
          tmem_ld32(T_O + lane_off + cc * 32, t);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
          tmem_st32(T_O + lane_off + cc * 32, t);
        }
        tmem_st_wait();
      }
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        const uint4 v4 = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        *reinterpret_cast<uint4*>(sm.p + swz_off(r, q * 8)) = v4;
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&sm.p_full);
    }
    if (ok) ok = warp_wait(&sm.o_full, (n_kv - 1) & 1, abort_flag);
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
      const int tok = q0 + r;
      const bool valid = tok < doc_end;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t t[32];
        tmem_ld32(T_O + lane_off + cc * 32, t);
        tmem_ld_wait();
        if (valid) {
          __nv_bfloat16* dst = out + static_cast<long long>(tok) * (Hq * DH) + h * DH + cc * 32;
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            uint4 v4;
            v4.x = pack_bf16x2(__uint_as_float(t[g8 * 8 + 0]) * inv_l, __uint_as_float(t[g8 * 8 + 1]) * inv_l);
            v4.y = pack_bf16x2(__uint_as_float(t[g8 * 8 + 2]) * inv_l, __uint_as_float(t[g8 * 8 + 3]) * inv_l);
            v4.z = pack_bf16x2(__uint_as_float(t[g8 * 8 + 4]) * inv_l, __uint_as_float(t[g8 * 8 + 5]) * inv_l);
            v4.w = pack_bf16x2(__uint_as_float(t[g8 * 8 + 6]) * inv_l, __uint_as_float(t[g8 * 8 + 7]) * inv_l);
            reinterpret_cast<uint4*>(dst)[g8] = v4;
          }
        }
      }
      if (valid) lse[static_cast<long long>(h) * T + tok] = m * scale + logf(l);
      tc_fence_before();
    } else if (lane == 0) {
      atomicCAS(status, 0, ST_TIMEOUT_TMEM_FULL);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ===================================================================== backward
struct BwdSmem {
  uint8_t k[TILE];
  uint8_t v[TILE];
  uint8_t q[TILE];
  uint8_t d_o[TILE];
  uint8_t pt[TILE];
  uint8_t dst[TILE];
  float lse2[128];
  float delta[128];
  uint64_t kv_full, qdo_full, qdo_empty, sdp_full, pds_full, dq_full, dq_done, ld_full;
  uint32_t tmem_ptr;
  int abort_flag;
};

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int T, int Hq) {
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;  // one warp per (t, h)
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(T) * Hq) return;
  const long long t = gw / Hq;
  const int h = static_cast<int>(gw % Hq);
  const long long off = (t * Hq + h) * DH + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(o + off);
  const uint2 b = *reinterpret_cast<const uint2*>(d_o + off);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
  const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
  for (int o2 = 16; o2 > 0; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

// dqkv[t, h*128 + d] = bf16(dq_acc[t, h*128 + d]) for the q heads
__global__ void attn_dq_convert_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, long long T,
                                       int Hq, int Hkv) {
  const long long qw = static_cast<long long>(Hq) * DH;
  const long long row = static_cast<long long>(Hq + 2 * Hkv) * DH;
  const long long total = T * qw / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * 4;
    const long long t = e / qw, cidx = e % qw;
    const float4 v = *reinterpret_cast<const float4*>(dq_acc + e);
    uint2 pk;
    pk.x = pack_bf16x2(v.x, v.y);
    pk.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dqkv + t * row + cidx) = pk;
  }
}


__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                const int* __restrict__ cu, int B, int Hq, int Hkv, const float* __restrict__ lse,
                const float* __restrict__ delta, float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, int T,
                float scale, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int doc_start, doc_end, kvb, ntiles;
  if (!find_tile(cu, B, blockIdx.x, doc_start, doc_end, kvb, ntiles)) return;  // kvb ascending: heaviest first
  const int kvh = blockIdx.y;
  const int G = Hq / Hkv;
  const int k0 = doc_start + kvb * TK;
  const int n_q = ntiles - kvb;  // query tiles kvb .. ntiles-1
  const int iters = G * n_q;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(&sm.kv_full, 1);
    mbar_init(&sm.qdo_full, 1);
    mbar_init(&sm.qdo_empty, 1);
    mbar_init(&sm.sdp_full, 1);
    mbar_init(&sm.pds_full, 256);
    mbar_init(&sm.dq_full, 1);
    mbar_init(&sm.dq_done, 8);
    mbar_init(&sm.ld_full, 128);
    sm.abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_ptr;
  const uint32_t T_ST = tmem, T_DPT = tmem + 128, T_DV = tmem + 256, T_DK = tmem + 384;
  const int kcol = (Hq + kvh) * DH, vcol = (Hq + Hkv + kvh) * DH;

  if (warp == 0) {
    if (elect_one()) {
      prefetch_tensormap(&tm_qkv);
      prefetch_tensormap(&tm_do);
      mbar_expect_tx(&sm.kv_full, 2 * TILE);
      tma_load_2d(sm.k, &tm_qkv, &sm.kv_full, kcol, k0);
      tma_load_2d(sm.k + SUB, &tm_qkv, &sm.kv_full, kcol + 64, k0);
      tma_load_2d(sm.v, &tm_qkv, &sm.kv_full, vcol, k0);
      tma_load_2d(sm.v + SUB, &tm_qkv, &sm.kv_full, vcol + 64, k0);
      for (int it = 0; it < iters; ++it) {
        const int h = kvh * G + it / n_q;
        const int q0 = doc_start + (kvb + it % n_q) * TQ;
        if (!mbar_wait(&sm.qdo_empty, (it & 1) ^ 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_EMPTY); break; }
        mbar_expect_tx(&sm.qdo_full, 2 * TILE);
        tma_load_2d(sm.q, &tm_qkv, &sm.qdo_full, h * DH, q0);
        tma_load_2d(sm.q + SUB, &tm_qkv, &sm.qdo_full, h * DH + 64, q0);
        tma_load_2d(sm.d_o, &tm_do, &sm.qdo_full, h * DH, q0);
        tma_load_2d(sm.d_o + SUB, &tm_do, &sm.qdo_full, h * DH + 64, q0);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t id_kk = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t id_kmn = umma_idesc_bf16(128, 128, false, true);
      constexpr uint32_t id_mnmn = umma_idesc_bf16(128, 128, true, true);
      const uint32_t k_a = smem_u32(sm.k), v_a = smem_u32(sm.v), q_a = smem_u32(sm.q), do_a = smem_u32(sm.d_o),
                     pt_a = smem_u32(sm.pt), ds_a = smem_u32(sm.dst);
      bool ok = mbar_wait(&sm.kv_full, 0, abort_flag);
      if (!ok) atomicCAS(status, 0, ST_TIMEOUT_FULL);
      for (int it = 0; it < iters && ok; ++it) {
        if (!mbar_wait(&sm.qdo_full, it & 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_FULL); break; }
        if (it > 0 && !mbar_wait(&sm.dq_done, (it - 1) & 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_TMEM_EMPTY); break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(T_ST, desc_kmajor(k_a, k), desc_kmajor(q_a, k), id_kk, k != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(T_DPT, desc_kmajor(v_a, k), desc_kmajor(do_a, k), id_kk, k != 0);
        umma_commit(&sm.sdp_full);
        if (!mbar_wait(&sm.pds_full, it & 1, abort_flag)) { atomicCAS(status, 0, ST_TIMEOUT_TMEM_EMPTY); break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(T_DV, desc_kmajor(pt_a, k), desc_mnmajor(do_a, k), id_kmn, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(T_DK, desc_kmajor(ds_a, k), desc_mnmajor(q_a, k), id_kmn, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_ss(T_ST, desc_mnmajor(ds_a, k), desc_mnmajor(k_a, k), id_mnmn, k != 0);
        umma_commit(&sm.qdo_empty);
        umma_commit(&sm.dq_full);
      }
    }
  } else {
    const int lane_grp = warp & 3;
    const int half = (warp - 2) >> 2;    // which 64 of the 128 columns this warp handles (same TMEM lanes as its twin)
    const int r = lane_grp * 32 + lane;  // key row for S^T / dK / dV; query row for the dQ tile
    const int tid = r;
    const uint32_t lane_off = static_cast<uint32_t>(lane_grp * 32) << 16;
    const float c = scale * LOG2E;
    const int key = k0 + r;
    bool ok = true;
    for (int it = 0; it < iters; ++it) {
      const int h = kvh * G + it / n_q;
      const int qt = kvb + it % n_q;
      const int q0 = doc_start + qt * TQ;
      const bool diag = (qt == kvb);
      if (half == 0) {
        const int tq = q0 + tid;
        const bool v = tq < doc_end;
        // every thread finished reading the previous iteration's values before pds_full
        // completed, and nobody passes dq_full before that, so overwriting here is safe
        sm.lse2[tid] = v ? lse[static_cast<long long>(h) * T + tq] * LOG2E : INFINITY;
        sm.delta[tid] = v ? delta[static_cast<long long>(h) * T + tq] : 0.f;
        mbar_arrive(&sm.ld_full);
      }
      ok = warp_wait(&sm.ld_full, it & 1, abort_flag);
      if (!ok) break;
      ok = warp_wait(&sm.sdp_full, it & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t s2[2][32], dp2[2][32];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        tmem_ld32(T_ST + lane_off + (half * 2 + u) * 32, s2[u]);
        tmem_ld32(T_DPT + lane_off + (half * 2 + u) * 32, dp2[u]);
      }
      tmem_ld_wait();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int cc = half * 2 + u;
        const uint32_t(&s)[32] = s2[u];
        const uint32_t(&dp)[32] = dp2[u];
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          float p[8], ds[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int qc = cc * 32 + g8 * 8 + i;  // query column
            float pv = ex2_approx(fmaf(__uint_as_float(s[g8 * 8 + i]), c, -sm.lse2[qc]));
            if (diag && r > qc) pv = 0.f;  // key after query
            p[i] = pv;
            ds[i] = pv * (__uint_as_float(dp[g8 * 8 + i]) - sm.delta[qc]) * scale;
          }
          uint4 a, b;
          a.x = pack_bf16x2(p[0], p[1]); a.y = pack_bf16x2(p[2], p[3]);
          a.z = pack_bf16x2(p[4], p[5]); a.w = pack_bf16x2(p[6], p[7]);
          b.x = pack_bf16x2(ds[0], ds[1]); b.y = pack_bf16x2(ds[2], ds[3]);
          b.z = pack_bf16x2(ds[4], ds[5]); b.w = pack_bf16x2(ds[6], ds[7]);
          const uint32_t off = swz_off(r, cc * 32 + g8 * 8);
          *reinterpret_cast<uint4*>(sm.pt + off) = a;
          *reinterpret_cast<uint4*>(sm.dst + off) = b;
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&sm.pds_full);
      ok = warp_wait(&sm.dq_full, it & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      {
        const int tq = q0 + r;
        const bool v = tq < doc_end;
        float* dst = dq_acc + static_cast<long long>(tq) * (Hq * DH) + h * DH;
        // dQ tile -> global accumulator.  A thread holds 64 columns of ONE query row; reduced directly, each 16-byte
        // reduction of a warp would hit a different row (half-used 32-byte sectors at the L2 atomic units).  Each warp
        // therefore transposes its 32 x 64 fp32 block through its own 8 KB slice of the P^T / dS^T buffers (free between
        // the MMAs that read them and the next iteration's writes, which wait for every warp's dq_done below) and issues
        // reductions that cover 256 contiguous bytes of a row.
        uint32_t t2[2][32];
#pragma unroll
        for (int u = 0; u < 2; ++u) tmem_ld32(T_ST + lane_off + (half * 2 + u) * 32, t2[u]);
        tmem_ld_wait();
        uint8_t* stg = sm.pt + (warp - 2) * (32 * 256);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int chunk = u * 8 + j;
            uint4 q4 = make_uint4(t2[u][4 * j], t2[u][4 * j + 1], t2[u][4 * j + 2], t2[u][4 * j + 3]);
            if (!v) q4 = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(stg + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = q4;
          }
        }
        __syncwarp();
        const int sub = lane >> 4, chunk = lane & 15;
        const int q_row0 = q0 + lane_grp * 32;
        float* base = dq_acc + static_cast<long long>(h) * DH + half * 64 + chunk * 4;
#pragma unroll 4
        for (int i = 0; i < 32; i += 2) {
          const int rr = i + sub;
          const int tok = q_row0 + rr;
          const uint4 u4 = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((chunk ^ (rr & 15)) << 4));
          if (tok < doc_end)
            red_add_v4(base + static_cast<long long>(tok) * (Hq * DH), __uint_as_float(u4.x), __uint_as_float(u4.y), __uint_as_float(u4.z),
                       __uint_as_float(u4.w));
        }
        (void)dst;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.dq_done);
    }
    if (ok) {
      // the last dq_full wait covers every MMA issued before it, including all dK/dV updates
      tc_fence_after();
      const bool v = key < doc_end;
      const long long row = static_cast<long long>(Hq + 2 * Hkv) * DH;
      {
        const int which = half;  // first column half of the warps writes dK, the second dV
        const uint32_t tbase = (which == 0 ? T_DK : T_DV) + lane_off;
        __nv_bfloat16* dst = dqkv + static_cast<long long>(key) * row + (which == 0 ? kcol : vcol);
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t t[32];
          tmem_ld32(tbase + cc * 32, t);
          tmem_ld_wait();
          if (v) {
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              uint4 pk;
              pk.x = pack_bf16x2(__uint_as_float(t[g8 * 8 + 0]), __uint_as_float(t[g8 * 8 + 1]));
              pk.y = pack_bf16x2(__uint_as_float(t[g8 * 8 + 2]), __uint_as_float(t[g8 * 8 + 3]));
              pk.z = pack_bf16x2(__uint_as_float(t[g8 * 8 + 4]), __uint_as_float(t[g8 * 8 + 5]));
              pk.w = pack_bf16x2(__uint_as_float(t[g8 * 8 + 6]), __uint_as_float(t[g8 * 8 + 7]));
              reinterpret_cast<uint4*>(dst + cc * 32)[g8] = pk;
            }
          }
        }
      }
      tc_fence_before();
    } else if (lane == 0) {
      atomicCAS(status, 0, ST_TIMEOUT_TMEM_FULL);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace b200

using namespace b200;

static int attn_tmap(CUtensorMap* m, const void* p, long long T, long long width) {
  return make_tmap_2d(m, p, static_cast<uint64_t>(T), static_cast<uint64_t>(width), static_cast<uint64_t>(width), 128, 64, 2,
                      true);
}

// qkv [T, (Hq+2Hkv)*128] bf16; cu_seqlens [B+1] int32 (device); out [T, Hq*128] bf16; lse [Hq, T] fp32.
extern "C" int b200_attn_fwd(const void* qkv, const int* cu_seqlens, void* out, float* lse, int* status, int T, int B,
                             int Hq, int Hkv, int Dh, int max_tiles, float scale, void* stream) {
  if (T <= 0 || B <= 0) return 0;
  if (Dh != DH || Hq % Hkv) return -1;
  CUtensorMap tm;
  int r = attn_tmap(&tm, qkv, T, static_cast<long long>(Hq + 2 * Hkv) * DH);
  if (r) return 10000 + r;
  const int smem = sizeof(FwdSmem) + 1024;
  static std::atomic<unsigned long long> cfg{0};
  {
    cudaError_t e = opt_in_shared_memory(attn_fwd_kernel, smem, cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid(max_tiles, Hq);
  attn_fwd_kernel<<<grid, ATT_THREADS, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      tm, cu_seqlens, B, Hq, Hkv, reinterpret_cast<__nv_bfloat16*>(out), lse, T, scale, status);
  return static_cast<int>(cudaGetLastError());
}

// scratch layout (caller-allocated, 16-byte aligned, (T*Hq*128 + Hq*T) floats):
// [dq_acc: T*Hq*128][delta: Hq*T] - dq_acc first so that its 16-byte vector reductions stay aligned

// d_out [T, Hq*128] bf16 -> dqkv [T, (Hq+2Hkv)*128] bf16 (every element written for rows < T).
extern "C" int b200_attn_bwd(const void* qkv, const void* out, const void* d_out, const float* lse,
                             const int* cu_seqlens, void* dqkv, void* scratch, int* status, int T, int B, int Hq,
                             int Hkv, int Dh, int max_tiles, float scale, void* stream) {
  if (T <= 0 || B <= 0) return 0;
  if (Dh != DH || Hq % Hkv) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float* dq_acc = reinterpret_cast<float*>(scratch);
  float* delta = dq_acc + static_cast<long long>(T) * Hq * DH;
  cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(T) * Hq * DH * sizeof(float), st);
  {
    const long long warps = static_cast<long long>(T) * Hq;
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    attn_delta_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                              reinterpret_cast<const __nv_bfloat16*>(d_out), delta, T, Hq);
  }
  CUtensorMap tq, tdo;
  int r = attn_tmap(&tq, qkv, T, static_cast<long long>(Hq + 2 * Hkv) * DH);
  if (r) return 10000 + r;
  r = attn_tmap(&tdo, d_out, T, static_cast<long long>(Hq) * DH);
  if (r) return 20000 + r;
  const int smem = sizeof(BwdSmem) + 1024;
  static std::atomic<unsigned long long> cfg{0};
  {
    cudaError_t e = opt_in_shared_memory(attn_bwd_kernel, smem, cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid(max_tiles, Hkv);
  attn_bwd_kernel<<<grid, BWD_THREADS, smem, st>>>(tq, tdo, cu_seqlens, B, Hq, Hkv, lse, delta, dq_acc,
                                                   reinterpret_cast<__nv_bfloat16*>(dqkv), T, scale, status);
  attn_dq_convert_kernel<<<148 * 8, 256, 0, st>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dqkv), T, Hq, Hkv);
  return static_cast<int>(cudaGetLastError());
}
