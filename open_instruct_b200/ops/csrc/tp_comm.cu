// Tensor-parallel inference: the all-reduce that follows a row-parallel projection (o_proj, down_proj), fused with
// the residual add and the RMSNorm that consume it - one kernel instead of {all-reduce, add, norm}.
//
// Every rank's projection writes its partial [B, D] bf16 result into a symmetric buffer.  The kernel then
//   1. tells every peer "my partial for this epoch is complete" (flag store into the peers' signal pads),
//   2. waits, bounded, for the same flag from every peer,
//   3. per row: reads that row out of EVERY rank's buffer with 16-byte peer loads, sums in fp32 in rank order (so all
//      ranks get bitwise the same result), adds the residual stream, writes the new residual stream, and
//   4. normalises the row (RMSNorm with weight) for the next projection.
// One-shot (every rank reads everything) is bandwidth-optimal for two ranks and latency-optimal for decode-sized
// messages.  The caller alternates between two symmetric buffers: a buffer is rewritten by the projection of call
// n + 2, which a peer can only reach after this rank has signalled call n + 1, i.e. after it finished reading here.
// All remote traffic is plain ld/st from the SMs; no TMA, no multicast.
#include "common.cuh"
#include "peer.cuh"

namespace b200 {

constexpr int PAD_TP_FLAG = 1100;  // [+rank]

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    acc[2 * k] += __uint_as_float(w[k] << 16);
    acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
  }
}

template <int NV>  // 16-byte vectors per thread: D <= NV * 256 * 8
__global__ void __launch_bounds__(256)
tp_allreduce_norm_kernel(PeerPtrs partials, PeerPtrs pads, int rank, int world, uint32_t epoch,
                         const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                         __nv_bfloat16* __restrict__ h_out, __nv_bfloat16* __restrict__ y_out, int B, int D, float eps,
                         long long limit_cycles, int* __restrict__ status) {
  __shared__ int peers_ok;
  __shared__ float red[8];
  if (threadIdx.x == 0) peers_ok = 1;
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(pads.p[threadIdx.x]) + PAD_TP_FLAG + rank, epoch);
  }
  __syncthreads();
  if (threadIdx.x < world && threadIdx.x != rank) {
    if (!wait_epoch(reinterpret_cast<const uint32_t*>(pads.p[rank]) + PAD_TP_FLAG + threadIdx.x, epoch, limit_cycles)) {
      atomicCAS(status, 0, ST_TIMEOUT_PEER);
      peers_ok = 0;
    }
  }
  __syncthreads();
  const bool remote = peers_ok != 0;  // after a timeout only the local partial is used; the status word tells the host
  const int nvec = D / 8;
  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * D;
    float acc[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = threadIdx.x + j * 256;
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[j][k] = 0.f;
      if (v < nvec) {
        if (residual) add_bf16x8(acc[j], *reinterpret_cast<const uint4*>(residual + base + v * 8));
#pragma unroll 1
        for (int r = 0; r < world; ++r) {
          if (r != rank && !remote) continue;
          add_bf16x8(acc[j], ld_volatile_u4(reinterpret_cast<const __nv_bfloat16*>(partials.p[r]) + base + v * 8));
        }
        uint4 pk;
        pk.x = pack_bf16x2(acc[j][0], acc[j][1]); pk.y = pack_bf16x2(acc[j][2], acc[j][3]);
        pk.z = pack_bf16x2(acc[j][4], acc[j][5]); pk.w = pack_bf16x2(acc[j][6], acc[j][7]);
        *reinterpret_cast<uint4*>(h_out + base + v * 8) = pk;
        // the norm sees the rounded residual stream, as a separate norm kernel reading h_out would
        const uint32_t q[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          acc[j][2 * k] = __uint_as_float(q[k] << 16);
          acc[j][2 * k + 1] = __uint_as_float(q[k] & 0xffff0000u);
          ss += acc[j][2 * k] * acc[j][2 * k] + acc[j][2 * k + 1] * acc[j][2 * k + 1];
        }
      }
    }
    if (w == nullptr) continue;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += red[k];
    __syncthreads();
    const float rstd = rsqrtf(tot / D + eps);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = threadIdx.x + j * 256;
      if (v < nvec) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + v * 8);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint4 pk;
        uint32_t* o = &pk.x;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          o[k] = pack_bf16x2(acc[j][2 * k] * rstd * __uint_as_float(ww[k] << 16),
                             acc[j][2 * k + 1] * rstd * __uint_as_float(ww[k] & 0xffff0000u));
        *reinterpret_cast<uint4*>(y_out + base + v * 8) = pk;
      }
    }
  }
}

}  // namespace b200

using namespace b200;

// partial_ptrs[r]: rank r's [B, D] bf16 partial (symmetric buffer, same offset on every rank).  residual / w may be
// null (no residual add / no norm).  h_out may alias residual.  D % 8 == 0, D <= 8192.
extern "C" int b200_tp_allreduce_norm(const void* const* partial_ptrs, const void* const* pad_ptrs, int rank, int world,
                                      unsigned epoch, const void* residual, const void* w, void* h_out, void* y_out, int B,
                                      int D, float eps, int limit_ms, int* status, void* stream) {
  if (world > MAX_PEERS || D % 8 || D > 8192 || B <= 0) return -1;
  const long long cycles = static_cast<long long>(limit_ms) * 1900000LL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = B < 148 * 4 ? B : 148 * 4;
  auto R = reinterpret_cast<const __nv_bfloat16*>(residual);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto H = reinterpret_cast<__nv_bfloat16*>(h_out);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y_out);
  const PeerPtrs pp = make_ptrs(partial_ptrs, world), pd = make_ptrs(pad_ptrs, world);
  if (D <= 2048) tp_allreduce_norm_kernel<1><<<grid, 256, 0, st>>>(pp, pd, rank, world, epoch, R, W, H, Y, B, D, eps, cycles, status);
  else if (D <= 4096) tp_allreduce_norm_kernel<2><<<grid, 256, 0, st>>>(pp, pd, rank, world, epoch, R, W, H, Y, B, D, eps, cycles, status);
  else tp_allreduce_norm_kernel<4><<<grid, 256, 0, st>>>(pp, pd, rank, world, epoch, R, W, H, Y, B, D, eps, cycles, status);
  return static_cast<int>(cudaGetLastError());
}
