// Helpers shared by the kernels that talk to peer GPUs through symmetric memory: peer pointer tables, signal-pad
// slots, system-scope flag stores/loads and the bounded epoch wait.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int MAX_PEERS = 8;
struct PeerPtrs {
  void* p[MAX_PEERS];
};

// signal-pad slots (uint32 index from the pad base); torch's own channels live below 1024
constexpr int PAD_BARRIER = 1024;       // [+rank]
constexpr int PAD_SCALAR_FLAG = 1040;   // [+rank]
constexpr int PAD_SCALAR_VAL = 1056;    // [+parity*8 + rank] (float bits)
constexpr int PAD_VEC_FLAG = 1136;      // [+rank]: small-vector all-reduce (metrics)
constexpr int PAD_BARRIER_SIDE = 1120;  // [+rank]; 1100..1107 is the tensor-parallel flag row (tp_comm.cu)

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
// wait until *addr has reached `epoch` (wrap-safe); false when the time limit ran out
__device__ __forceinline__ bool wait_epoch(const uint32_t* addr, uint32_t epoch, long long limit_cycles) {
  const long long t0 = clock64();
  while (static_cast<int32_t>(ld_acquire_sys(addr) - epoch) < 0) {
    if (clock64() - t0 > limit_cycles) return false;
    __nanosleep(64);
  }
  return true;
}

// 16-byte load that is never served from a stale L1 line (peer buffers are rewritten between launches)
__device__ __forceinline__ uint4 ld_volatile_u4(const void* addr) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr) : "memory");
  return v;
}

static inline PeerPtrs make_ptrs(const void* const* host, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_PEERS; ++i) pp.p[i] = i < world ? const_cast<void*>(host[i]) : nullptr;
  return pp;
}

}  // namespace b200
