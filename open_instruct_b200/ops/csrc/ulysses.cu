// Sequence parallelism (Ulysses): the head -> sequence exchange as one kernel of peer stores.
//
// Before attention every rank holds ALL tokens for ITS heads; after attention each rank needs ITS tokens for ALL heads.
// `a2a_heads_kernel` walks this rank's [T, n_blocks * 128] matrix and stores rows [j * T_l, (j + 1) * T_l) into rank j's
// buffer, 128-column head block b landing at column `dst_col[b]` there (16-byte stores straight into peer memory).  The
// opposite direction (sequence -> head) needs no kernel of its own: it is the column-scatter epilogue of the projection
// GEMM that produces the data (gemm2.cu).  The same kernel returns dQ/dK/dV to the token owners in the backward pass.
#include "common.cuh"
#include "peer.cuh"

namespace b200 {

__global__ void __launch_bounds__(256)
a2a_heads_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src, PeerPtrs dsts, long long ld_dst,
                 const int* __restrict__ dst_col, int T, int T_l, int n_blocks) {
  // one 16-byte vector = 8 bf16; a 128-column block has 16 vectors
  const long long total = static_cast<long long>(T) * n_blocks * 16;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vec = static_cast<int>(i & 15);
    const long long rb = i >> 4;
    const int blk = static_cast<int>(rb % n_blocks);
    const int row = static_cast<int>(rb / n_blocks);
    const int dst_rank = row / T_l;
    const int dst_row = row - dst_rank * T_l;
    const uint4 v = *reinterpret_cast<const uint4*>(src + row * ld_src + blk * 128 + vec * 8);
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dsts.p[dst_rank]) + dst_row * ld_dst + dst_col[blk] + vec * 8) = v;
  }
  __threadfence_system();
}

}  // namespace b200

using namespace b200;

// src: [T, n_blocks * 128] bf16 (row stride ld_src); dst_ptrs[j]: rank j's [T_l, *] bf16 buffer (row stride ld_dst);
// dst_col: device int[n_blocks].  T == world * T_l.
extern "C" int b200_a2a_heads(const void* src, long long ld_src, const void* const* dst_ptrs, int world, long long ld_dst,
                              const int* dst_col, int T, int T_l, int n_blocks, void* stream) {
  if (world > MAX_PEERS || T != world * T_l || ld_src % 8 || ld_dst % 8) return -1;
  if (T == 0 || n_blocks == 0) return 0;
  a2a_heads_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), ld_src, make_ptrs(dst_ptrs, world), ld_dst, dst_col, T, T_l, n_blocks);
  return static_cast<int>(cudaGetLastError());
}
