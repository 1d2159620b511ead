// Dense bf16/fp16 GEMM on CTA pairs: two SMs work on one 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// A cluster of two CTAs is the unit of work. Each CTA loads its own 128 rows of A and its own 128 of the 256 B rows
// (columns of C) per K block - 32 KB per stage instead of the 48 KB a lone CTA needs for a 128 x 256 tile, so the same
// shared memory holds five stages and two output staging buffers per epilogue group and every byte fetched from L2 feeds 1.5x the FLOPs. The even CTA of the pair (the
// leader) issues the MMAs; the instruction reads both CTAs' shared memory and writes each CTA's half of the
// accumulator (its 128 rows x 256 columns) into that CTA's TMEM. Each CTA drains its own half through the same fused
// epilogue as the single-CTA kernel.
//
// Barriers (per stage unless noted):
//   full   - in the leader only, count 1: the leader's producer arrives with the byte count of BOTH CTAs' copies; the
//            peer's TMA loads complete their bytes on the leader's barrier (cp.async.bulk.tensor ... cta_group::2 with a
//            shared::cluster barrier address). No load here uses cluster multicast.
//   empty  - in both CTAs, count 1: tcgen05.commit.cta_group::2 with multicast to both CTAs releases the stage in each.
//   tmem_full[2]  - in both CTAs, count 1: multicast commit after the last K block of a tile.
//   tmem_empty[2] - in the leader, count 512: the 256 epilogue threads of each CTA arrive (the peer's remotely).
// Every wait is bounded (two seconds of %globaltimer); a CTA that gives up reports through the status word, waits
// for the copies it issued and still meets its peer at the closing cluster barrier, so neither CTA leaves while the
// other can still touch its shared memory or barriers.
//
// Covers the same reference family as the single-CTA kernel (gemm_tc_{nn,nt,tn,tt}_f32 with bias / GELU / GELU-grad /
// residual epilogues, src/Idrak.Gpu/Cuda/PtxKernels.TensorCore.cs:24-29,80-144) for the large-M products of a
// training step.
#include "gemm_epilogue.cuh"
#include <cstdlib>
#include <cstring>

namespace idrak {

constexpr int kPairBN = 256;        // columns of the pair's tile; each CTA stages half of the B rows
constexpr int kHalfBN = 128;

struct PairSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kHalfBN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;       // 32 KB
  static constexpr int kStages = 5;
  static constexpr int kStagingBytes = 2 * kDenseStagingBytes;   // two buffers per epilogue group
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};
static_assert(PairSmem::kTotal <= 232448, "shared memory per CTA");

// ---------------------------------------------------------------------------------------------------------------
// cluster / cta_group::2 wrappers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_shared_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A tiled load into this CTA's shared memory whose bytes complete on a barrier given by its shared::cluster address
// (the leader's). No multicast: the data lands in the issuing CTA only.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `mask` once the MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}
__device__ __forceinline__ void tc_mma_pair_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// the kernel: grid = 2 x pairs, cluster (2, 1, 1); warp roles as in the single-CTA kernel
// ---------------------------------------------------------------------------------------------------------------
template <int A_MN, int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kDenseThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux, const GemmParams p) {
  using L = PairSmem;
  constexpr int kStages = L::kStages;
  constexpr int BN = kPairBN;
  extern __shared__ uint8_t smem_raw[];
  // the same offsets in both CTAs: the MMA applies one descriptor to both
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + kStages * L::kStageBytes;
  uint8_t* bar_base = staging + L::kStagingBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();          // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;
  const int k_blocks = (p.K + kBK - 1) / kBK;
  const int units = p.m_tiles * p.n_tiles;           // tiles of 256 x 256

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2 * 32 * kEpiWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 2 * BN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs have their barriers and TMEM before either signals the other
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = pair; unit < units && ok; unit += pairs) {
        int tm, tn, split;
        unit_to_tile(p, unit, tm, tn, split);
        const int row0 = tm * 2 * kBM + int(rank) * kBM;          // this CTA's rows of A
        const int col0 = tn * BN + int(rank) * kHalfBN;           // this CTA's rows of B
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (2u << 16) | stage)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          const uint32_t bar = map_shared_to_cta(smem_u32(&full[stage]), 0);
          if (leader) mbar_expect_tx(&full[stage], 2 * L::kStageBytes);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmA, bar, row0 + j * 64, kb * kBK);
          } else {
            tma_load_2d_pair(sa, &tmA, bar, kb * kBK, row0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < kHalfBN / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmB, bar, col0 + j * 64, kb * kBK);
          } else {
            tma_load_2d_pair(sb, &tmB, bar, kb * kBK, col0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok || *abort_flag) {
        // the copies this CTA issued complete on the leader's barrier, which the peer cannot poll: give them time to
        // land (they take microseconds) before the closing barrier lets shared memory go
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) { }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * kBM, BN, A_MN, B_MN, 1);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      unsigned long long t_acc = 0, t_ops = 0;
      const long long t_begin = p.prof ? clock64() : 0;
      for (int unit = pair; unit < units && ok; unit += pairs, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        const long long c0 = p.prof ? clock64() : 0;
        if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag, p.st, kTimeoutTmemEmpty, (2u << 16) | buf)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (p.prof) t_acc += (unsigned long long)(clock64() - c0);
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          const long long c2 = p.prof ? clock64() : 0;
          if (!mbar_wait(&full[stage], phase, abort_flag, p.st, kTimeoutSmemFull, (2u << 16) | stage)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (p.prof) t_ops += (unsigned long long)(clock64() - c2);
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sb + kk * 32, 16, 1024);
            tc_mma_pair_f16_ss(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit_pair(&empty[stage], 0x3);     // both CTAs may refill the stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit_pair(&tmem_full[buf], 0x3);
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 0] = (unsigned long long)(clock64() - t_begin);
        p.prof[blockIdx.x * 8 + 1] = t_acc;
        p.prof[blockIdx.x * 8 + 2] = t_ops;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps, this CTA's 128 rows)
    const int ewarp = warp - 2;
    const uint32_t empty_bar_leader0 = map_shared_to_cta(smem_u32(&tmem_empty[0]), 0);
    const uint32_t empty_bar_leader1 = map_shared_to_cta(smem_u32(&tmem_empty[1]), 0);
    int local = 0;
    unsigned long long t_wait = 0, t_busy = 0;
    SideAhead ahead;
    ahead.ready = false;
    ahead.ring = 0;
    for (int unit = pair; unit < units; unit += pairs, ++local) {
      int tm, tn, split;
      unit_to_tile(p, unit, tm, tn, split);
      NextTile next{false, 0, 0};
      if (unit + pairs < units) {
        int nm, nn, ns;
        unit_to_tile(p, unit + pairs, nm, nn, ns);
        next = NextTile{true, nm * 2 * kBM + int(rank) * kBM, nn * BN};
      }
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const long long c0 = p.prof ? clock64() : 0;
      if (!mbar_wait(&tmem_full[buf], acc_phase, abort_flag, p.st, kTimeoutTmemFull, (2u << 16) | buf)) break;
      tc_fence_after();
      const long long c1 = p.prof ? clock64() : 0;
      uint64_t* done_local = &tmem_empty[buf];
      const uint32_t done_remote = buf ? empty_bar_leader1 : empty_bar_leader0;
      // this CTA's half of the accumulator is free once read: tell the leader's MMA warp
      drain_accumulator<BN, 2>(p, &tmC, &tmAux, tmem_base + buf * BN, ewarp, lane, tm * 2 * kBM + int(rank) * kBM, tn * BN,
                            0, true, staging, ahead, next, [=]() {
                              tc_fence_before();
                              if (leader) mbar_arrive(done_local);
                              else mbar_arrive_cluster(done_remote);
                            });
      if (p.prof) {
        t_wait += (unsigned long long)(c1 - c0);
        t_busy += (unsigned long long)(clock64() - c1);
      }
    }
    if (p.tma_store && (ewarp & 3) == 2 && lane == 0) tma_store_wait<0>();
    if (p.prof && ewarp == 0 && lane == 0) {
      p.prof[blockIdx.x * 8 + 4] = t_wait;
      p.prof[blockIdx.x * 8 + 5] = t_busy;
      p.prof[blockIdx.x * 8 + 6] = (unsigned long long)local;
    }
  }

  tc_fence_before();
  __syncthreads();
  // neither CTA leaves (or frees TMEM) while the other may still signal it or have MMAs reading its shared memory
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * BN);
  }
}

template <int A_MN, int B_MN>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmAux,
                       const GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kTotal));
      }))
    return e;
  kern<<<grid, kDenseThreads, PairSmem::kTotal, stream>>>(tmA, tmB, tmC, tmAux, p);
  note_launches(1);
  return int(cudaGetLastError());
}

static int pair_operand_map(CUtensorMap* tm, const void* ptr, int mn_extent, int k_extent, int ld, int mn_major, int fp16) {
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  if (mn_major) {
    dims[0] = uint64_t(mn_extent); dims[1] = uint64_t(k_extent);
    box[0] = 64; box[1] = kBK;
  } else {
    dims[0] = uint64_t(k_extent); dims[1] = uint64_t(mn_extent);
    box[0] = kBK; box[1] = 128;
  }
  strides[0] = uint64_t(ld) * 2;
  return encode_tensor_map(tm, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           const_cast<void*>(ptr), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Whether a product of this size goes to CTA pairs: enough 256 x 256 tiles to occupy most pairs, one K pass.
bool gemm_pair_wanted(int M, int N, int K, int splits) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("IDRAK_GEMM_PAIR");
    enabled = (e == nullptr) ? 1 : (e[0] == '0' ? 0 : (e[0] == '2' ? 2 : 1));     // 0 off, 1 where it measured faster, 2 wherever it can run
  }
  if (!enabled || splits > 1 || M < 1024 || N < 256 || K < 128) return false;
  const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
  if (tiles < sm_count() / 4) return false;
  // measured against the single-CTA kernel (cold L2, CUDA-graph replays): pairs win from K = 3072 (+13 %) and on very wide
  // outputs (+2..4 %), and lose ~5 % on K = 768 with modest N, where the tile's fixed costs dominate
  return enabled == 2 || K >= 2048 || N >= 16384;
}

// Same contract as the single-CTA launcher; `p` arrives filled except for the tile counts. tmC / tmAux are the store maps
// (box 64 x 128) made by the caller.
int gemm_pair_launch(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, const CUtensorMap& tmC,
                     const CUtensorMap& tmAux, GemmParams p, int fp16, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  if (pair_operand_map(&tmA, A, p.M, p.K, lda, a_mn, fp16)) return -11;
  if (pair_operand_map(&tmB, B, p.N, p.K, ldb, b_mn, fp16)) return -12;
  p.m_tiles = (p.M + 2 * kBM - 1) / (2 * kBM);
  p.n_tiles = (p.N + kPairBN - 1) / kPairBN;
  p.splits = 1;
  const int units = p.m_tiles * p.n_tiles;
  const int pairs = min(units, sm_count() / 2);
  const int grid = 2 * pairs;
  if (!a_mn && !b_mn) return launch_pair<0, 0>(tmA, tmB, tmC, tmAux, p, grid, stream);
  if (!a_mn && b_mn) return launch_pair<0, 1>(tmA, tmB, tmC, tmAux, p, grid, stream);
  if (a_mn && !b_mn) return launch_pair<1, 0>(tmA, tmB, tmC, tmAux, p, grid, stream);
  return launch_pair<1, 1>(tmA, tmB, tmC, tmAux, p, grid, stream);
}

}  // namespace idrak
