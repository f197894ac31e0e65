// bf16 GEMM for sm_100a on CTA PAIRS: tcgen05.mma.cta_group::2, 256x256 output tile per pair.
//
// Same contract as gemm.cu (C[M,N] (op)= A_op[M,K] * B_op[N,K]^T, K-major or MN-major operands,
// bf16 / fp32 / fp32-accumulate epilogues).  Two CTAs of a cluster share one tile:
//   * CTA r loads its own 128 rows of A and HALF of the B tile (128 of the 256 columns), so the
//     shared-memory fill per k-block drops from 48 KB to 32 KB per SM for the same tensor work;
//     that ratio, not the tensor pipe, is what limits the one-CTA kernel;
//   * every TMA load of both CTAs reports its bytes to the LEADER CTA's full barrier
//     (cp.async.bulk.tensor with .cta_group::2, no cluster broadcast form is used);
//   * the leader's elected thread issues tcgen05.mma.cta_group::2 (M = 256 split over the two
//     CTAs' tensor memories, N = 256) and commits completion to BOTH CTAs' barriers with two
//     plain commits (one per CTA);
//   * each CTA drains its own 128 x 256 fp32 accumulator; 2 accumulators per CTA (all 512 TMEM
//     columns) so the epilogue of tile i overlaps the main loop of tile i+1.
// 6 stages x 32 KB of shared memory per CTA.
#include <cooperative_groups.h>

#include "common.cuh"
#include "pair.cuh"

namespace b200 {
namespace g2 {

constexpr int BM = 128;        // rows per CTA (pair tile = 256)
constexpr int BN = 256;        // pair tile columns
constexpr int BNH = 128;       // B columns loaded by each CTA
constexpr int BK = 64, UK = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_BYTES = BNH * BK * 2;  // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int STAGING_BYTES = 4 * 32 * 256;  // scatter epilogue: per epilogue warp 32 rows x 128 bf16 columns
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256 + STAGING_BYTES;

// OUT_F32_RED accumulates like OUT_F32_ACC but with 16-byte `red.global.add` instead of load + add + store: the epilogue
// warps no longer wait on a DRAM round trip per row (the gradient buffer never sits in L2), the L2 does the addition.
enum OutMode : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2, OUT_F32_RED = 3 };

using namespace pair;

struct Sched {
  int num_m, num_n, total;  // in 256x256 pair tiles
  // Row tiles per sweep of the column tiles.  The A rows of a sweep are re-read for every column tile and must stay in
  // L2 (about 40 MB of its 126 are budgeted for them), while B is streamed once per sweep: the more row tiles a sweep
  // holds, the fewer times B comes from DRAM (gate/up forward at 4096 tokens: 4 sweeps -> 1, 1.08 GB -> 0.3 GB read).
  int group;
  __device__ __forceinline__ void set_group(int K, int N) {
    const long long bytes_per_row_tile = 2LL * BM * K * 2;
    const long long b_bytes = 2LL * N * K;
    // a B operand that fits in L2 stays there too: the sweep's A rows get what is left of about 56 MB
    long long budget = 40LL << 20;
    if (b_bytes <= (48LL << 20)) budget = (56LL << 20) - b_bytes;
    if (budget < (8LL << 20)) budget = 8LL << 20;
    const long long gmax = budget / bytes_per_row_tile;
    group = static_cast<int>(gmax < 4 ? 4 : (gmax > 64 ? 64 : gmax));
  }
  __device__ __forceinline__ void get(int t, int& m_blk, int& n_blk) const {
    const int GROUP = group;
    const int per_group = GROUP * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP;
    const int gsz = min(num_m - first_m, GROUP);
    const int r = t - g * per_group;
    m_blk = first_m + r % gsz;
    n_blk = r / gsz;
  }
};

template <bool A_MN, bool B_MN, int OUT>
__global__ void __launch_bounds__(THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
             void* __restrict__ Cout, int M, int N, int K, long long ldc, int* __restrict__ status,
             const long long* __restrict__ scatter, int row_off, const long long* __restrict__ scatter2) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                       // [STAGES]  used in the leader only
  uint64_t* empty = bars + STAGES;             // [STAGES]  one per CTA
  uint64_t* tfull = bars + 2 * STAGES;         // [2]       one per CTA
  uint64_t* tempty = bars + 2 * STAGES + 2;    // [2]       used in the leader only (8 arrivals)
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  uint8_t* staging = smem + STAGES * STAGE_BYTES + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  Sched sched;
  sched.num_m = (M + 2 * BM - 1) / (2 * BM);
  sched.num_n = (N + BN - 1) / BN;
  sched.total = sched.num_m * sched.num_n;
  sched.set_group(K, N);
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_ptr, 512);
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
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < sched.total && ok; t += num_pairs) {
        int m_blk, n_blk;
        sched.get(t, m_blk, n_blk);
        const int m0 = m_blk * 2 * BM + cta * BM;   // my rows of A / C
        const int n0 = n_blk * BN + cta * BNH;      // my half of the B tile
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            atomicCAS(status, 0, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          const uint32_t leader_full = mapa(smem_u32(&full[s]), 0);
          if (cta == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_BYTES;
          uint8_t* b_dst = sB + s * B_BYTES;
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, &tma_a, leader_full, k0, m0);
          } else {
#pragma unroll
            for (int b = 0; b < BM / 64; ++b) tma_load_2d_pair(a_dst + b * (BK * 128), &tma_a, leader_full, m0 + b * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(b_dst, &tma_b, leader_full, k0, n0);
          } else {
#pragma unroll
            for (int b = 0; b < BNH / 64; ++b) tma_load_2d_pair(b_dst + b * (BK * 128), &tma_b, leader_full, n0 + b * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int t = pair; t < sched.total && ok; t += num_pairs, ++tile_i) {
        const uint32_t acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag)) {
          atomicCAS(status, 0, ST_TIMEOUT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag)) {
            atomicCAS(status, 0, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t ad = A_MN ? umma_desc_sw128(a_addr + k * (UK * 128), BK * 128, 1024)
                                     : umma_desc_sw128(a_addr + k * (UK * 2), 16, 1024);
            const uint64_t bd = B_MN ? umma_desc_sw128(b_addr + k * (UK * 128), BK * 128, 1024)
                                     : umma_desc_sw128(b_addr + k * (UK * 2), 16, 1024);
            umma_ss_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // release this stage in both CTAs once the MMAs above have read it
          umma_commit_pair(mapa(smem_u32(&empty[s]), 0));
          umma_commit_pair(mapa(smem_u32(&empty[s]), 1));
        }
        if (ok) {
          umma_commit_pair(mapa(smem_u32(&tfull[acc]), 0));
          umma_commit_pair(mapa(smem_u32(&tfull[acc]), 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int lane_grp = warp & 3;
    uint32_t tile_i = 0;
    for (int t = pair; t < sched.total; t += num_pairs, ++tile_i) {
      int m_blk, n_blk;
      sched.get(t, m_blk, n_blk);
      const uint32_t acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (OUT == OUT_F32_ACC) {
        // the accumulate epilogue reads the old gradient tile, which never sits in L2 (the gradient buffer is streamed once
        // per micro-batch): ask L2 for this thread's row now, while the tile's MMAs are still running
        const int prow = m_blk * 2 * BM + cta * BM + lane_grp * 32 + lane;
        if (prow < M) {
          const char* pc = reinterpret_cast<const char*>(reinterpret_cast<const float*>(Cout) + static_cast<long long>(prow) * ldc + n_blk * BN);
          const int ncols = min(BN, N - n_blk * BN);
#pragma unroll
          for (int b = 0; b < BN * 4; b += 128)
            if (b < ncols * 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(pc + b));
        }
      }
      const bool ready = __all_sync(0xffffffffu, mbar_wait(&tfull[acc], acc_ph, abort_flag));
      if (!ready) {
        if (lane == 0) atomicCAS(status, 0, ST_TIMEOUT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const int row = m_blk * 2 * BM + cta * BM + lane_grp * 32 + lane;
      const int n0 = n_blk * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + acc * BN;
      if (OUT == OUT_BF16 && (scatter != nullptr || (N & 127) == 0)) {
        // Coalescing epilogue (also the scatter epilogue, whose destinations may be peer GPUs).  One TMEM lane per thread means
        // a thread holds one ROW; stored directly, every 16-byte store of a warp lands in a different row - tolerable for local
        // L2, wasteful over NVLink (measured 2.4x on a peer push).  So each warp transposes through shared memory: 32 rows x 128
        // columns are staged (16-byte chunks XOR-swizzled by row against bank conflicts) and written back two rows per
        // instruction, 256 contiguous bytes per row.  Used for every bf16 output whose width is a multiple of 128.  (The fp32
        // outputs keep the row-per-thread form: a thread already moves whole 128-byte lines there, and the transposed
        // read-modify-write measured 30 % slower because its loads are no longer all in flight at once.)
        uint8_t* stg = staging + lane_grp * (32 * 256);
        const int row0 = m_blk * 2 * BM + cta * BM + lane_grp * 32;
#pragma unroll 1
        for (int hb = 0; hb < BN / 128; ++hb) {
          const int col0 = n0 + hb * 128;
          if (col0 >= N) break;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(taddr + hb * 128 + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              const int chunk = c * 4 + j;  // 16-byte chunk of this thread's 256-byte row
              *reinterpret_cast<uint4*>(stg + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = v;
            }
          }
          __syncwarp();
          __nv_bfloat16* d1 = scatter ? reinterpret_cast<__nv_bfloat16*>(scatter[col0 >> 7]) : reinterpret_cast<__nv_bfloat16*>(Cout) + col0;
          __nv_bfloat16* d2 = scatter2 ? reinterpret_cast<__nv_bfloat16*>(scatter2[col0 >> 7]) : nullptr;
          const int sub = lane >> 4, chunk = lane & 15;
#pragma unroll 4
          for (int i = 0; i < 32; i += 2) {
            const int rr = i + sub;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((chunk ^ (rr & 15)) << 4));
            const int grow = row0 + rr;
            if (grow < M) {
              const long long off = static_cast<long long>(grow + row_off) * ldc + chunk * 8;
              *reinterpret_cast<uint4*>(d1 + off) = v;
              if (d2) *reinterpret_cast<uint4*>(d2 + off) = v;
            }
          }
          __syncwarp();
        }
      } else if ((OUT == OUT_F32 || OUT == OUT_F32_ACC) && (N & 63) == 0) {
        // Coalescing fp32 epilogue.  Row-per-thread stores cost the fp32 modes a sixth of the kernel's rate even without the
        // read (measured: bf16 output 0.98 of peak, fp32 store-only 0.82): a warp's 16-byte stores land in 32 different rows,
        // so every 32-byte sector is written in two halves by two instructions.  Here each warp stages 32 rows x 64 columns
        // through shared memory (16-byte chunks XOR-swizzled by row) and writes rows back whole: 16 lanes x 16 bytes = 256
        // contiguous bytes, two rows per instruction.  In accumulate mode the 16 loads of the old values of a thread are
        // issued BEFORE the accumulator is read from tensor memory, so all of them are in flight while it is staged.
        uint8_t* stg = staging + lane_grp * (32 * 256);
        const int row0 = m_blk * 2 * BM + cta * BM + lane_grp * 32;
        const int sub = lane >> 4, chunk = lane & 15;
#pragma unroll 1
        for (int qb = 0; qb < BN / 64; ++qb) {
          const int col0 = n0 + qb * 64;
          if (col0 >= N) break;
          float* cbase = reinterpret_cast<float*>(Cout) + col0 + chunk * 4;
          float4 old[16];
          if (OUT == OUT_F32_ACC) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int grow = row0 + 2 * i + sub;
              if (grow < M) old[i] = *reinterpret_cast<const float4*>(cbase + static_cast<long long>(grow) * ldc);
            }
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld32(taddr + qb * 64 + h * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int ch = h * 8 + j;  // 16-byte chunk of this thread's 256-byte staged row
              *reinterpret_cast<uint4*>(stg + lane * 256 + ((ch ^ (lane & 15)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int rr = 2 * i + sub;
            float4 v = *reinterpret_cast<const float4*>(stg + rr * 256 + ((chunk ^ (rr & 15)) << 4));
            const int grow = row0 + rr;
            if (grow < M) {
              if (OUT == OUT_F32_ACC) { v.x += old[i].x; v.y += old[i].y; v.z += old[i].z; v.w += old[i].w; }
              *reinterpret_cast<float4*>(cbase + static_cast<long long>(grow) * ldc) = v;
            }
          }
          __syncwarp();
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col = n0 + c * 32;
        if (col >= N) break;
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row < M) {
          if (OUT == OUT_BF16) {
            // column scatter: every 128-column block has its own destination base (possibly in a peer GPU's memory),
            // rows shift by row_off; used to fuse the sequence -> head exchange into the projection
            __nv_bfloat16* crow =
                scatter ? reinterpret_cast<__nv_bfloat16*>(scatter[col >> 7]) + static_cast<long long>(row + row_off) * ldc + (col & 127)
                        : reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<long long>(row) * ldc + col;
            if (col + 32 <= N) {
              // second destination table: the same tile also goes to another buffer (a peer GPU's copy), so that a
              // tensor-parallel partial result reaches every rank while the following tiles are still being computed
              __nv_bfloat16* crow2 =
                  scatter2 ? reinterpret_cast<__nv_bfloat16*>(scatter2[col >> 7]) + static_cast<long long>(row + row_off) * ldc + (col & 127)
                           : nullptr;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                reinterpret_cast<uint4*>(crow)[j] = v;
                if (crow2) reinterpret_cast<uint4*>(crow2)[j] = v;
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
      if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&tempty[acc]), 0));  // leader counts 4 warps x 2 CTAs
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
  }
  cluster_sync();  // neither CTA leaves while its partner may still signal into it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

static int max_pairs_cache = 0;

template <bool A_MN, bool B_MN, int OUT>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc,
                  int* status, cudaStream_t stream, int max_ctas, const long long* scatter = nullptr, int row_off = 0,
                  const long long* scatter2 = nullptr) {
  auto kern = gemm2_kernel<A_MN, B_MN, OUT>;
  static std::atomic<unsigned long long> configured{0};
  {
    cudaError_t e = opt_in_shared_memory(kern, SMEM, configured);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!max_pairs_cache) {
    int n = 0;
    cfg.gridDim = dim3(148);
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = 64;
    max_pairs_cache = n;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  int pairs = tiles < max_pairs_cache ? tiles : max_pairs_cache;
  if (max_ctas > 1 && pairs > max_ctas / 2) pairs = max_ctas / 2;
  cfg.gridDim = dim3(2 * pairs);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, C, M, N, K, ldc, status, scatter, row_off, scatter2);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

}  // namespace g2
}  // namespace b200

// Same arguments as b200_gemm_bf16 (see gemm.cu); runs the CTA-pair kernel.
extern "C" int b200_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                               long long ldc, int a_mn, int b_mn, int out_mode, int* status, void* stream,
                               int max_ctas) {
  using namespace b200;
  using namespace b200::g2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  else r = make_tmap_2d(&ta, A, K, M, lda, BK, 64, 2, true);
  if (r) return 10000 + r;
  if (!b_mn) r = make_tmap_2d(&tb, B, N, K, ldb, BNH, BK, 2, true);
  else r = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2, true);
  if (r) return 20000 + r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define B200_DISPATCH2(AM, BMN)                                                                              \
  switch (out_mode) {                                                                                         \
    case 0: return g2::launch<AM, BMN, g2::OUT_BF16>(ta, tb, C, M, N, K, ldc, status, st, max_ctas);          \
    case 1: return g2::launch<AM, BMN, g2::OUT_F32>(ta, tb, C, M, N, K, ldc, status, st, max_ctas);           \
    case 2: return g2::launch<AM, BMN, g2::OUT_F32_ACC>(ta, tb, C, M, N, K, ldc, status, st, max_ctas);       \
    case 3: return g2::launch<AM, BMN, g2::OUT_F32_RED>(ta, tb, C, M, N, K, ldc, status, st, max_ctas);       \
    default: return -2;                                                                                       \
  }
  if (!a_mn && !b_mn) { B200_DISPATCH2(false, false) }
  if (!a_mn && b_mn) { B200_DISPATCH2(false, true) }
  if (a_mn && !b_mn) { B200_DISPATCH2(true, false) }
  B200_DISPATCH2(true, true)
#undef B200_DISPATCH2
}

// C is not one matrix: column block j (128 wide) of the bf16 result goes to `scatter[j]` (device table of base
// addresses, local or peer memory) at row `row + row_off`, leading dimension `ld_dst`.  N % 128 == 0.
// `scatter2` (optional): a second table of the same shape; every tile is stored to both destinations.
extern "C" int b200_gemm2_bf16_scatter(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                       int a_mn, int b_mn, const long long* scatter, int row_off, long long ld_dst,
                                       int* status, void* stream, const long long* scatter2) {
  using namespace b200;
  using namespace b200::g2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (N % 128 || scatter == nullptr) return -3;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d(&ta, A, M, K, lda, BM, BK, 2, true);
  else r = make_tmap_2d(&ta, A, K, M, lda, BK, 64, 2, true);
  if (r) return 10000 + r;
  if (!b_mn) r = make_tmap_2d(&tb, B, N, K, ldb, BNH, BK, 2, true);
  else r = make_tmap_2d(&tb, B, K, N, ldb, BK, 64, 2, true);
  if (r) return 20000 + r;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return g2::launch<false, false, g2::OUT_BF16>(ta, tb, nullptr, M, N, K, ld_dst, status, st, 0, scatter, row_off, scatter2);
  if (!a_mn && b_mn) return g2::launch<false, true, g2::OUT_BF16>(ta, tb, nullptr, M, N, K, ld_dst, status, st, 0, scatter, row_off, scatter2);
  if (a_mn && !b_mn) return g2::launch<true, false, g2::OUT_BF16>(ta, tb, nullptr, M, N, K, ld_dst, status, st, 0, scatter, row_off, scatter2);
  return g2::launch<true, true, g2::OUT_BF16>(ta, tb, nullptr, M, N, K, ld_dst, status, st, 0, scatter, row_off, scatter2);
}
