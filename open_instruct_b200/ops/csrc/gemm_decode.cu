// Decode-sized GEMM for sm_100a: C[M, N] = A[M, K] * W[N, K]^T with M <= 256 rows (one row per running sequence).
//
// With so few rows the product is a stream over the weights, and what limits it is how evenly and how thinly that stream
// is spread over the SMs: measured on the 8B shapes at M = 256, the general kernels ran with the SMs busy 53-70 % of the
// time (wave quantisation: 112 tiles on 74 CTA pairs, 96 tiles on 148 SMs) at about 80 GB/s per busy SM, with neither HBM
// (27-51 %) nor L2 (26-36 %) saturated.  (A read-only stream tops out near 3.9 TB/s on this GPU - a library reduction over
// 2 GiB measures 3.88, a fill 3.91, a copy 6.56 with half the bytes in each direction - so that, not the copy figure, is
// the ceiling of a weight stream.)  So this kernel is shaped by two rules:
//   * ONE wave: the caller picks the tile width (BNS columns per MMA, NSUB MMAs side by side, up to 448 columns) and a
//     K split so that (column tiles x K slices) is at most the number of CTA pairs, every pair getting an equal slice;
//   * few bytes into each SM: a CTA pair covers all 256 rows (tcgen05.mma.cta_group::2, each CTA loads its own 128 rows of A
//     and half of each B tile), so the activations cross L2 -> SM once per column tile per CTA, not once per 128 x 128 tile.
// A K-split launch writes fp32 partial tiles to `S` planes with plain stores (no atomics: the result does not depend on
// the order in which CTAs finish); the consumer (the fused add + RMSNorm that follows o_proj / down_proj) sums the planes.
//
// Warps: 0 = TMA producer (both CTAs), 1 = MMA issuer (leader CTA), 2-5 = epilogue (TMEM -> registers -> global).
// Every wait is bounded (mbar_wait) and reports through the status word.
#include "common.cuh"
#include "pair.cuh"

namespace b200 {
namespace gd {

using namespace pair;

constexpr int BM = 128;  // rows per CTA (pair tile = 256 rows)
constexpr int BK = 64, UK = 16;
constexpr int A_BYTES = BM * BK * 2;  // 16 KB
constexpr int THREADS = 192;
constexpr int SMEM_LIMIT = 232448;    // 227 KB of dynamic shared memory per CTA

template <int BNS, int NSUB>
struct Cfg {
  static_assert(BNS % 32 == 0 && BNS >= 32 && BNS <= 256, "MMA width: a multiple of 32 up to 256");
  static_assert(NSUB == 1 || NSUB == 2, "one or two MMAs side by side");
  static_assert(BNS * NSUB <= 512, "accumulators must fit the 512 tensor-memory columns");
  static constexpr int BNT = BNS * NSUB;            // columns per pair tile
  static constexpr int B_ROWS = BNS / 2;            // rows of each B sub-tile held by one CTA
  static constexpr int B_BYTES = B_ROWS * BK * 2;   // a multiple of 1024 (B_ROWS is a multiple of 16)
  static constexpr int STAGE_BYTES = A_BYTES + NSUB * B_BYTES;
  static constexpr int STAGES_FIT = (SMEM_LIMIT - 1024 - 512) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 512;
  static constexpr int TMEM_COLS = BNT <= 64 ? 64 : (BNT <= 128 ? 128 : (BNT <= 256 ? 256 : 512));
};

// grid = 2 * n_tiles * splits CTAs in clusters of 2.  `C`: bf16 [M, N] (OUT32 = false, splits must be 1) or fp32 planes
// [splits][M][N] with row stride ldc and plane stride `plane` elements (OUT32 = true).
template <int BNS, int NSUB, bool OUT32>
__global__ void __launch_bounds__(THREADS, 1)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, void* __restrict__ Cout,
                   int M, int N, int K, long long ldc, long long plane, int n_tiles, int kb_per_split, int* __restrict__ status) {
  using C = Cfg<BNS, NSUB>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES] used in the leader only: both CTAs' loads report their bytes here
  uint64_t* empty = bars + C::STAGES;       // [STAGES] one per CTA
  uint64_t* tfull = bars + 2 * C::STAGES;   // [1]      one per CTA
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int n_tile = pair_id % n_tiles, ks = pair_id / n_tiles;
  const int num_kb = (K + BK - 1) / BK;
  const int kb0 = ks * kb_per_split, kb1 = min(num_kb, kb0 + kb_per_split);
  const int n_base = n_tile * C::BNT;

  griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(tfull, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_ptr, C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync();  // both CTAs' barriers are initialised before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      prefetch_tensormap(&tma_a);
      prefetch_tensormap(&tma_b);
      // (Requesting several K blocks of a row back to back, to give HBM longer contiguous runs, was measured and changed
      // nothing: 65.5 us with one block per turn, 67.8 / 68.6 us with groups of 2 / 4 on the gate/up shape.)
      //
      // The weights do not depend on the kernel before this one, the activations do: the B tiles of the first ring turn are
      // requested right away (under programmatic dependent launch that is while the predecessor still runs), the A tiles
      // after the grid dependency has resolved.  Both halves of a stage report to the same barrier.
      const int pre = min(C::STAGES, kb1 - kb0);
      for (int i = 0; i < pre; ++i) {
        const uint32_t leader_full = mapa(smem_u32(&full[i]), 0);
        if (cta == 0) mbar_expect_tx(&full[i], 2 * C::STAGE_BYTES);
        uint8_t* st = smem + i * C::STAGE_BYTES;
#pragma unroll
        for (int j = 0; j < NSUB; ++j)
          tma_load_2d_pair(st + A_BYTES + j * C::B_BYTES, &tma_b, leader_full, (kb0 + i) * BK, n_base + j * BNS + static_cast<int>(cta) * C::B_ROWS);
      }
      griddep_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d_pair(smem + i * C::STAGE_BYTES, &tma_a, mapa(smem_u32(&full[i]), 0), (kb0 + i) * BK, static_cast<int>(cta) * BM);
      uint32_t it = pre;
      for (int kb = kb0 + pre; kb < kb1; ++kb, ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
          atomicCAS(status, 0, ST_TIMEOUT_EMPTY);
          break;
        }
        const uint32_t leader_full = mapa(smem_u32(&full[s]), 0);
        if (cta == 0) mbar_expect_tx(&full[s], 2 * C::STAGE_BYTES);
        uint8_t* st = smem + s * C::STAGE_BYTES;
        const int k0 = kb * BK;
        tma_load_2d_pair(st, &tma_a, leader_full, k0, static_cast<int>(cta) * BM);
#pragma unroll
        for (int j = 0; j < NSUB; ++j)
          tma_load_2d_pair(st + A_BYTES + j * C::B_BYTES, &tma_b, leader_full, k0, n_base + j * BNS + static_cast<int>(cta) * C::B_ROWS);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BNS, false, false);
      uint32_t it = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1;
        if (!mbar_wait(&full[s], ph, abort_flag)) {
          atomicCAS(status, 0, ST_TIMEOUT_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
#pragma unroll
        for (int j = 0; j < NSUB; ++j) {
          const uint32_t b_addr = a_addr + A_BYTES + j * C::B_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t ad = umma_desc_sw128(a_addr + k * (UK * 2), 16, 1024);
            const uint64_t bd = umma_desc_sw128(b_addr + k * (UK * 2), 16, 1024);
            umma_ss_pair(tmem_base + j * BNS, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
        }
        // release this stage in both CTAs once the MMAs above have read it
        umma_commit_pair(mapa(smem_u32(&empty[s]), 0));
        umma_commit_pair(mapa(smem_u32(&empty[s]), 1));
      }
      if (ok) {
        umma_commit_pair(mapa(smem_u32(tfull), 0));
        umma_commit_pair(mapa(smem_u32(tfull), 1));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int lane_grp = warp & 3;  // the TMEM lane quarter this warp may read
    griddep_wait();  // stores below must not overtake the predecessor (they could not anyway: the accumulator needs A)
    const bool ready = __all_sync(0xffffffffu, mbar_wait(tfull, 0, abort_flag));
    if (!ready) {
      if (lane == 0) atomicCAS(status, 0, ST_TIMEOUT_TMEM_FULL);
    } else {
      tc_fence_after();
      const int row = static_cast<int>(cta) * BM + lane_grp * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < C::BNT / 16; ++c) {
        const int col = n_base + c * 16;
        if (col >= N) break;  // warp-uniform: whole 16-column groups (N is a multiple of 16)
        uint32_t r[16];
        tmem_ld16(taddr + c * 16, r);
        tmem_ld_wait();
        if (row < M) {
          if (OUT32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(Cout) + ks * plane + static_cast<long long>(row) * ldc + col);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              dst[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                                   __uint_as_float(r[4 * q + 3]));
          } else {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<long long>(row) * ldc + col);
#pragma unroll
            for (int q = 0; q < 2; ++q)
              dst[q] = make_uint4(pack_bf16x2(__uint_as_float(r[8 * q]), __uint_as_float(r[8 * q + 1])),
                                  pack_bf16x2(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3])),
                                  pack_bf16x2(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5])),
                                  pack_bf16x2(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7])));
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give TMA copies that may still be in flight time to land before the CTA's shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
  }
  cluster_sync();  // neither CTA leaves while its partner may still signal into it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

template <int BNS, int NSUB, bool OUT32>
static int launch(const void* A, const void* W, void* Cout, int M, int N, int K, long long lda, long long ldb, long long ldc,
                  long long plane, int splits, int* status, cudaStream_t stream) {
  using C = Cfg<BNS, NSUB>;
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  if (r) return 10000 + r;
  r = make_tmap_2d(&tb, W, N, K, ldb, C::B_ROWS, BK, 2, true);
  if (r) return 20000 + r;
  auto kern = gemm_decode_kernel<BNS, NSUB, OUT32>;
  static std::atomic<unsigned long long> configured{0};
  {
    cudaError_t e = opt_in_shared_memory(kern, C::SMEM, configured);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int num_kb = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > num_kb) splits = num_kb;
  int per = (num_kb + splits - 1) / splits;
  while (splits > 1 && per * (splits - 1) >= num_kb) {  // no empty K slice: every plane the consumer sums is written
    --splits;
    per = (num_kb + splits - 1) / splits;
  }
  const int n_tiles = (N + C::BNT - 1) / C::BNT;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: this kernel may start (prologue + first weight tiles) while its predecessor finishes
  const bool pdl = pdl_enabled();
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(THREADS);
  cfg.gridDim = dim3(2 * n_tiles * splits);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, Cout, M, N, K, ldc, plane, n_tiles, per, status);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gd
}  // namespace b200

// C = A[M, K] * W[N, K]^T for M <= 256 (bf16 operands, K-major, 16-byte aligned rows; N a multiple of 16).
//   bns, nsub : tile shape, one of (64,1) (96,1) (128,1) (256,1) (192,2) (224,2) (256,2)
//   splits = 1: C is bf16 [M, N] with row stride ldc.
//   splits > 1: C is fp32 [splits][M][N] (row stride ldc, plane stride `plane` floats); plane s receives the product over
//               the s-th K slice (slices of ceil(K/64 / splits) 64-wide blocks; the count is lowered when a slice would
//               be empty, so the caller computes the same count before sizing C).  Only (128,1), (256,1), (256,2).
// Returns 0, a CUDA / driver error, -1 (M > 256 or N % 16), -2 (unsupported tile shape for this output).
extern "C" int b200_gemm_decode(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldb,
                                long long ldc, long long plane, int bns, int nsub, int splits, int* status, void* stream) {
  using namespace b200::gd;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 256 || (N & 15)) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int key = bns * 10 + nsub;
  if (splits <= 1) {
    switch (key) {
      case 641: return launch<64, 1, false>(A, W, C, M, N, K, lda, ldb, ldc, 0, 1, status, st);
      case 961: return launch<96, 1, false>(A, W, C, M, N, K, lda, ldb, ldc, 0, 1, status, st);
      case 1281: return launch<128, 1, false>(A, W, C, M, N, K, lda, ldb, ldc, 0, 1, status, st);
      case 2561: return launch<256, 1, false>(A, W, C, M, N, K, lda, ldb, ldc, 0, 1, status, st);
      case 1922: return launch<192, 2, false>(A, W, C, M, N, K, lda, ldb, ldc, 0, 1, status, st);
      case 2242: return launch<224, 2, false>(A, W, C, M, N, K, lda, ldb, ldc, 0, 1, status, st);
      case 2562: return launch<256, 2, false>(A, W, C, M, N, K, lda, ldb, ldc, 0, 1, status, st);
      default: return -2;
    }
  }
  switch (key) {
    case 1281: return launch<128, 1, true>(A, W, C, M, N, K, lda, ldb, ldc, plane, splits, status, st);
    case 2561: return launch<256, 1, true>(A, W, C, M, N, K, lda, ldb, ldc, plane, splits, status, st);
    case 2562: return launch<256, 2, true>(A, W, C, M, N, K, lda, ldb, ldc, plane, splits, status, st);
    default: return -2;
  }
}
