// Shared pieces of the peer-memory kernels: the context a kernel receives (peer flag areas, exchange slots,
// epoch word), system-scope flag stores / loads, bounded waits on peers and the "last block" counter.
#pragma once
#include "common.cuh"

namespace idrak {

constexpr int kMaxRanks = 8;
constexpr int kFlagChannels = 512;

struct CommCtx {
  int rank, world;
  uint32_t* flags[kMaxRanks];    // flags[p] = rank p's flag area: [kFlagChannels][kMaxRanks] words
  float* slots[kMaxRanks];       // slots[p] = rank p's small-value exchange area: [kMaxRanks][slot_floats]
  int slot_floats;
  uint32_t* epoch;               // device word: current step epoch (monotone)
  uint32_t* counters;            // device words: "last block" counters, one per channel
  Status* st;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread t < world publishes `value` on `channel` to peer t.
__device__ __forceinline__ void signal_peers(const CommCtx& c, int channel, uint32_t value) {
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + channel * kMaxRanks + c.rank, value);
  }
}

// Every thread returns true once all peers (except `skip`, if given) published >= value on `channel` (bounded).
__device__ __forceinline__ bool wait_peers(const CommCtx& c, int channel, uint32_t value, uint32_t kernel_id,
                                           int skip = -1) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < c.world && int(threadIdx.x) != skip) {
    const uint32_t* f = c.flags[c.rank] + channel * kMaxRanks + threadIdx.x;
    uint64_t t0 = 0;
    uint32_t polls = 0;
    while (int32_t(ld_acquire_sys(f) - value) < 0) {
      if ((++polls & 63u) == 0u) {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > IDRAK_WAIT_BUDGET_NS) {
          report(c.st, kTimeoutPeerFlag, (kernel_id << 16) | (uint32_t(channel) << 4) | threadIdx.x, value);
          ok_flag = 0;
          break;
        }
      }
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

// Returns true in every thread of the last block of the grid to arrive (all other blocks' stores are visible).
__device__ __forceinline__ bool last_block(const CommCtx& c, int counter) {
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t n = atomicAdd(c.counters + counter, 1u);
    is_last = (n == gridDim.x - 1);
    if (is_last) c.counters[counter] = 0;   // ready for the next launch
  }
  __syncthreads();
  return is_last != 0;
}

__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  return __ldcg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ void accum_bf16x8(float (&acc)[8], uint4 v, float w) {
  float2 f;
  f = unpack_bf16x2(v.x); acc[0] += w * f.x; acc[1] += w * f.y;
  f = unpack_bf16x2(v.y); acc[2] += w * f.x; acc[3] += w * f.y;
  f = unpack_bf16x2(v.z); acc[4] += w * f.x; acc[5] += w * f.y;
  f = unpack_bf16x2(v.w); acc[6] += w * f.x; acc[7] += w * f.y;
}


}  // namespace idrak
