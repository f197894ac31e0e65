// bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   C[M,N] (op)= A_op[M,K] * B_op[N,K]^T        fp32 accumulation in tensor memory
//
// Operands may be stored K-major ([rows, K], K contiguous) or MN-major ([K, rows], rows
// contiguous); the three GEMMs of a linear layer map onto this without any transpose copy:
//   forward  y  = x W^T      : A = x  (K-major),  B = W  (K-major)
//   dgrad    dx = dy W       : A = dy (K-major),  B = W  (MN-major, reduction over W's rows)
//   wgrad    dW += dy^T x    : A = dy (MN-major), B = x  (MN-major), fp32 accumulate epilogue
//
// One persistent CTA per SM, 6 warps: warp 0 issues TMA loads into a 4-stage ring, warp 1
// issues tcgen05.mma (one elected thread) into one of two 128x256 fp32 accumulators (all 512
// TMEM columns), warps 2-5 drain the other accumulator with tcgen05.ld, so the epilogue of
// tile i overlaps the main loop of tile i+1.
#include "common.cuh"

namespace b200 {

constexpr int BM = 128, BN = 256, BK = 64, UK = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_SMEM = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /*align*/ + 256 /*barriers*/;

enum OutMode : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2, OUT_F32_RED = 3 /* atomic fp32 add: split-K partial sums */ };

struct TileSched {
  int num_m, num_n, total;
  __device__ __forceinline__ void get(int t, int& m_blk, int& n_blk) const {
    // groups of 8 row-blocks sweep the column blocks, so concurrently resident CTAs share
    // A rows and B columns through L2
    constexpr int GROUP = 8;
    const int per_group = GROUP * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP;
    const int gsz = min(num_m - first_m, GROUP);
    const int r = t - g * per_group;
    m_blk = first_m + r % gsz;
    n_blk = r / gsz;
  }
};

template <bool A_MN, bool B_MN, int OUT, int BN_T = BN, int STAGES_T = STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 void* __restrict__ Cout, int M, int N, int K, long long ldc, int* __restrict__ status, int splits) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES_T * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES_T * (A_STAGE_BYTES + (BN_T * BK * 2)));
  uint64_t* full = bars;                 // [STAGES_T]
  uint64_t* empty = bars + STAGES_T;       // [STAGES_T]
  uint64_t* tfull = bars + 2 * STAGES_T;   // [2]
  uint64_t* tempty = bars + 2 * STAGES_T + 2;  // [2]
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * STAGES_T + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  TileSched sched;
  sched.num_m = (M + BM - 1) / BM;
  sched.num_n = (N + BN_T - 1) / BN_T;
  const int tiles = sched.num_m * sched.num_n;
  sched.total = tiles * splits;  // work item t: output tile t / splits, K slice t % splits (split-K: partial sums are added atomically)
  const int num_kb = (K + BK - 1) / BK;
  const int kb_per = (num_kb + splits - 1) / splits;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES_T; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      prefetch_tensormap(&tma_a);
      prefetch_tensormap(&tma_b);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
        int m_blk, n_blk;
        sched.get(t / splits, m_blk, n_blk);
        const int m0 = m_blk * BM, n0 = n_blk * BN_T;
        const int kb0 = (t % splits) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES_T;
          const uint32_t ph = (it / STAGES_T) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            atomicCAS(status, 0, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], A_STAGE_BYTES + (BN_T * BK * 2));
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * (BN_T * BK * 2);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(a_dst, &tma_a, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int b = 0; b < BM / 64; ++b) tma_load_2d(a_dst + b * (BK * 128), &tma_a, &full[s], m0 + b * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tma_b, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int b = 0; b < BN_T / 64; ++b) tma_load_2d(b_dst + b * (BK * 128), &tma_b, &full[s], n0 + b * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN_T, A_MN, B_MN);
      uint32_t it = 0;
      uint32_t tile_i = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x, ++tile_i) {
        const uint32_t acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag)) {
          atomicCAS(status, 0, ST_TIMEOUT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN_T;
        const int kb0 = (t % splits) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES_T;
          const uint32_t ph = (it / STAGES_T) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag)) {
            atomicCAS(status, 0, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * (BN_T * BK * 2));
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // K-major: advance 16 elements (32 B) inside the 128 B swizzle row;
            // MN-major: advance 16 K-rows of 128 B.
            const uint64_t ad = A_MN ? umma_desc_sw128(a_addr + k * (UK * 128), BK * 128, 1024)
                                     : umma_desc_sw128(a_addr + k * (UK * 2), 16, 1024);
            const uint64_t bd = B_MN ? umma_desc_sw128(b_addr + k * (UK * 128), BK * 128, 1024)
                                     : umma_desc_sw128(b_addr + k * (UK * 2), 16, 1024);
            umma_ss(d_tmem, ad, bd, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // stage reusable once these MMAs have read it
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int lane_grp = warp & 3;  // TMEM lanes this warp may touch: 32*lane_grp .. +31
    uint32_t tile_i = 0;
    for (int t = blockIdx.x; t < sched.total; t += gridDim.x, ++tile_i) {
      int m_blk, n_blk;
      sched.get(t / splits, m_blk, n_blk);
      const uint32_t acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      // the decision must be warp-uniform: the TMEM loads below are .sync.aligned
      const bool ready = __all_sync(0xffffffffu, mbar_wait(&tfull[acc], acc_ph, abort_flag));
      if (!ready) {
        if (lane == 0) atomicCAS(status, 0, ST_TIMEOUT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const int row = m_blk * BM + lane_grp * 32 + lane;
      const int n0 = n_blk * BN_T;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + acc * BN_T;
#pragma unroll 1
      for (int c = 0; c < BN_T / 32; ++c) {
        const int col = n0 + c * 32;
        if (col >= N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row < M) {
          if (OUT == OUT_BF16) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<long long>(row) * ldc + col;
            if (col + 32 <= N) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                reinterpret_cast<uint4*>(crow)[j] = v;
              }
            } else {
              for (int j = 0; j < 32 && col + j < N; ++j) crow[j] = __float2bfloat16(__uint_as_float(r[j]));
            }
          } else {
            float* crow = reinterpret_cast<float*>(Cout) + static_cast<long long>(row) * ldc + col;
            if (col + 32 <= N) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (OUT == OUT_F32_RED) {
                  red_add_v4(crow + 4 * j, v.x, v.y, v.z, v.w);
                  continue;
                }
                if (OUT == OUT_F32_ACC) {
                  const float4 o = reinterpret_cast<float4*>(crow)[j];
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                reinterpret_cast<float4*>(crow)[j] = v;
              }
            } else {
              for (int j = 0; j < 32 && col + j < N; ++j) {
                float v = __uint_as_float(r[j]);
                if (OUT == OUT_F32_RED) {
                  atomicAdd(crow + j, v);
                  continue;
                }
                if (OUT == OUT_F32_ACC) v += crow[j];
                crow[j] = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give TMA copies that may still be in flight time to land before the CTA's shared
    // memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------- host
EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tmap_2d(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                 uint32_t box_cols, int elem_bytes, bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <bool A_MN, bool B_MN, int OUT, int BN_T = BN, int STAGES_T = STAGES>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc,
                  int* status, cudaStream_t stream, int max_ctas, int splits = 1) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, OUT, BN_T, STAGES_T>;
  constexpr int smem = STAGES_T * (A_STAGE_BYTES + BN_T * BK * 2) + 1024 /*align*/ + 256 /*barriers*/;
  static std::atomic<unsigned long long> configured{0};
  {
    cudaError_t e = opt_in_shared_memory(kern, smem, configured);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int num_kb = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > num_kb) splits = num_kb;
  while (splits > 1 && ((num_kb + splits - 1) / splits) * (splits - 1) >= num_kb) --splits;  // no empty K slice
  const int tiles = ((M + BM - 1) / BM) * ((N + BN_T - 1) / BN_T) * splits;
  int grid = tiles < num_sms() ? tiles : num_sms();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  kern<<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, C, M, N, K, ldc, status, splits);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace b200

// C[M,N] (op)= A_op[M,K] * B_op[N,K]^T.
//   a_mn = 0: A stored [M,K] (row stride lda);  a_mn = 1: A stored [K,M] (row stride lda)
//   b_mn = 0: B stored [N,K] (row stride ldb);  b_mn = 1: B stored [K,N] (row stride ldb)
//   out_mode: 0 = bf16 store, 1 = fp32 store, 2 = fp32 accumulate (C += A*B)
// `status` is a device int the kernel sets non-zero when a bounded wait ran out.
// Returns 0 or a CUDA/driver error code. Alignment: base pointers 16 B, lda/ldb/ldc multiples of 8.
extern "C" int b200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                              long long ldb, long long ldc, int a_mn, int b_mn, int out_mode, int* status,
                              void* stream, int max_ctas) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  else r = make_tmap_2d(&ta, A, K, M, lda, BK, 64, 2, true);
  if (r) return 10000 + r;
  if (!b_mn) r = make_tmap_2d(&tb, B, N, K, ldb, BN, BK, 2, true);
  else r = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2, true);
  if (r) return 20000 + r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define B200_DISPATCH(AM, BMN)                                                                              \
  switch (out_mode) {                                                                                        \
    case 0: return launch<AM, BMN, OUT_BF16>(ta, tb, C, M, N, K, ldc, status, st, max_ctas);                 \
    case 1: return launch<AM, BMN, OUT_F32>(ta, tb, C, M, N, K, ldc, status, st, max_ctas);                  \
    case 2: return launch<AM, BMN, OUT_F32_ACC>(ta, tb, C, M, N, K, ldc, status, st, max_ctas);              \
    default: return -2;                                                                                      \
  }
  if (!a_mn && !b_mn) { B200_DISPATCH(false, false) }
  if (!a_mn && b_mn) { B200_DISPATCH(false, true) }
  if (a_mn && !b_mn) { B200_DISPATCH(true, false) }
  B200_DISPATCH(true, true)
#undef B200_DISPATCH
}

// Narrow-tile variant for small M (decode): C[M,N] = A[M,K] * B[N,K]^T, bf16 out, 128 x 64 tiles and an 8-stage ring.
// With few rows the GEMM is a stream over the weights; 64-wide column tiles give 4x as many CTAs as the 256-wide
// kernel, so all SMs pull on HBM (M = 256, N = 4096: 128 CTAs instead of 32).
// `bn`: 64 (8-stage ring) or 128 (6-stage ring; half of every stage is weights instead of a third).
extern "C" int b200_gemm_bf16_skinny(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                     long long ldb, long long ldc, int* status, void* stream, int bn) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (bn != 64 && bn != 128) return -4;
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  if (r) return 10000 + r;
  r = make_tmap_2d(&tb, B, N, K, ldb, bn, BK, 2, true);
  if (r) return 20000 + r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 64) return launch<false, false, OUT_BF16, 64, 8>(ta, tb, C, M, N, K, ldc, status, st, 0);
  return launch<false, false, OUT_BF16, 128, 6>(ta, tb, C, M, N, K, ldc, status, st, 0);
}

// Split-K variant for small M and long K (decode-sized down / o projections): C32[M,N] += A[M,K] * B[N,K]^T with the K
// range cut into `splits` slices that run on different SMs and add their fp32 partial tiles atomically.  The caller zeroes
// C32 first (or seeds it with a residual) and converts afterwards.  128 x 128 tiles.
extern "C" int b200_gemm_bf16_splitk(const void* A, const void* B, float* C32, int M, int N, int K, long long lda,
                                     long long ldb, long long ldc, int splits, int* status, void* stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  if (r) return 10000 + r;
  r = make_tmap_2d(&tb, B, N, K, ldb, 128, BK, 2, true);
  if (r) return 20000 + r;
  return launch<false, false, OUT_F32_RED, 128, 6>(ta, tb, C32, M, N, K, ldc, status, reinterpret_cast<cudaStream_t>(stream), 0, splits);
}
