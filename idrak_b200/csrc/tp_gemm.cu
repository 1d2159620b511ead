// Tensor-parallel linear layers as ONE kernel each: the tcgen05 GEMM and the collective that goes with it run
// together, tile by tile, over NVLink peer memory.
//
//   mode 1  all-gather -> GEMM   (column-parallel layer with row-sharded activations)
//           Every rank holds rows [rank * R, (rank + 1) * R) of X. A few CTAs of the kernel push this rank's rows
//           into every peer's gather buffer (plain 16-byte stores, nearest-following peer first) and publish one
//           flag per 128-row chunk; the other CTAs are the persistent GEMM over Y[M, N_local] = X · W_local^T and
//           start with the rows that are already there (own rows, then rank-1, rank-2, ... in arrival order),
//           waiting on the chunk's flag right before its first TMA load.
//   mode 2  GEMM -> reduce-scatter   (row-parallel layer)
//           P = X_local[M, K_local] · W_local^T is a partial sum of the full output. The epilogue stores each
//           128-row tile straight into its owner's staging slot [this rank] (coalesced 128-byte rows through a
//           shared-memory slab), rows of rank+1 first and own rows last, and the last tile of a chunk publishes
//           the chunk's flag on the owner. When a CTA runs out of tiles it turns reducer: it waits for a chunk's
//           flags from all ranks and sums the W slots in rank order (fp32), adds bias / residual and writes the
//           rank's own rows. The order is fixed, so every run gives the same bits.
//
// Ordering between ranks: one device counter `seq` numbers the fused ops of a rank (all ranks issue the same ops
// in the same order). Op q uses half (q & 1) of the gather / staging buffers, publishes flags with value q + 1,
// and at its end publishes "done = q + 1" to all peers; a writer waits for done >= q - 1 from its target before
// touching a half (op q - 2 used it last). Nothing depends on the host: the kernels are graph-capturable.
// Every wait is bounded (two seconds) and reports (code, where) to the status word instead of hanging.
// No TMA load touches another GPU's memory and none uses multicast: peers are reached with ld / st only.
//
// The reference has no tensor parallelism (its cluster layer is data-parallel and pipeline,
// src/Idrak.Network/Training/*); the layer contracts these kernels serve are Linear.ForwardCore
// (src/Idrak/Layers/Linear.cs:165) and the collectives of src/Idrak.Abstraction/Cluster/Collectives.cs:34-80.
#include "comm.cuh"
#include "gemm_epilogue.cuh"
#include <cstring>

namespace idrak {

constexpr int kTpBN = 256;
constexpr int kTpStages = 4;
constexpr int kTpChDone = 440;         // flag channel: ops completed by a rank
constexpr int kTpChReady0 = 448;       // flag channels [448, 512): one per 128-row chunk of a rank's rows
constexpr int kTpMaxChunks = 64;

struct TpParams {
  int mode;                  // 1 all-gather -> GEMM, 2 GEMM -> reduce-scatter
  int rows_per_rank;         // multiple of 128
  int chunks_per_rank;
  int push_ctas;             // mode 1: CTAs [0, push_ctas) move rows instead of computing tiles
  int hold_done;             // 1: do not publish "done" at the end (the caller keeps reading the gathered rows)
  uint32_t* seq;             // device word: fused ops completed on this rank
  uint32_t* counters;        // device words: [0] CTAs finished, [1 + m_tile] tiles stored (mode 2)
  // mode 1
  const __nv_bfloat16* x_local;
  int ldx;
  __nv_bfloat16* gather[kMaxRanks];   // rank p's gather area: two halves of [M, K]
  long long gather_half;              // elements per half
  // mode 2
  __nv_bfloat16* stage[kMaxRanks];    // rank p's staging area: two halves of [world][rows_per_rank, N]
  long long stage_half;
  __nv_bfloat16* out;                 // [rows_per_rank, ldo]
  int ldo;
  const __nv_bfloat16* rs_residual;   // [rows_per_rank, rs_ldr] or null
  int rs_ldr;
  const __nv_bfloat16* rs_bias;       // [N] or null
  // NVSwitch multicast views of the same areas (null: plain peer stores / loads)
  __nv_bfloat16* gather_mc;           // a store here lands in every rank's gather area
  const __nv_bfloat16* stage_mc;      // a reducing load here sums every rank's staging area, laid out [M, N]
};

struct TpSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kTpBN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = 4 * 2 * 4096;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kTpStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

// One thread polls a flag of this rank's own flag area until it reaches `value` (wrap-safe compare).
__device__ __forceinline__ bool tp_poll(const uint32_t* f, uint32_t value, Status* st, uint32_t where) {
  uint64_t t0 = 0;
  uint32_t polls = 0;
  while (int32_t(ld_acquire_sys(f) - value) < 0) {
    if ((++polls & 63u) == 0u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > IDRAK_WAIT_BUDGET_NS) {
        report(st, kTimeoutPeerFlag, where, value);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Barrier over the 128 epilogue threads that also ORs a predicate: every thread learns whether any of them
// failed, so they all leave a loop together and nobody is left waiting at a later barrier.
__device__ __forceinline__ bool epi_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(uint32_t(pred))
      : "memory");
  return r != 0;
}

// 16-byte store through an NVSwitch multicast address: the switch writes it into every rank's copy.
__device__ __forceinline__ void multimem_st16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// 16-byte load through a multicast address that returns the sum over every rank's copy (8 bf16 values, summed
// in fp32 inside the switch).
__device__ __forceinline__ uint4 multimem_ld_reduce16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ __forceinline__ void tp_unit_to_tile(const GemmParams& p, const TpParams& t, const CommCtx& c, int unit,
                                                int& tm, int& tn, int& owner, int& chunk) {
  const int per_owner = t.chunks_per_rank * p.n_tiles;
  const int oi = unit / per_owner;
  const int r = unit - oi * per_owner;
  // inside an owner's block the row chunks vary fastest: the CTAs working side by side share one tile of W, which
  // is then read from DRAM once per owner instead of once per chunk
  tn = r / t.chunks_per_rank;
  chunk = r - tn * t.chunks_per_rank;
  owner = (t.mode == 1) ? (c.rank - oi + c.world) % c.world : (c.rank + 1 + oi) % c.world;
  tm = owner * t.chunks_per_rank + chunk;
}

// mode 1, CTAs [0, push_ctas): copy this rank's rows into every rank's gather half and flag each chunk.
__device__ void tp_push_rows(const GemmParams& p, const TpParams& t, const CommCtx& c, uint32_t q) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {      // the half about to be overwritten was last read by op q - 2 of each target
    if (!tp_poll(c.flags[c.rank] + kTpChDone * kMaxRanks + threadIdx.x, q - 1u, c.st, (40u << 16) | threadIdx.x))
      ok_flag = 0;
  }
  __syncthreads();
  if (!ok_flag) return;
  const int row_vecs = p.K / 8;                                  // 16-byte vectors per row
  const long long half_off = (long long)(q & 1u) * t.gather_half;
  if (t.gather_mc != nullptr) {
    // NVSwitch multicast: one store per 16 bytes reaches every rank's gather buffer (own copy included), so this
    // rank's rows leave the GPU once instead of once per peer.
    // A chunk is cut into kParts row slabs so that every push CTA has work even with few chunks; the CTA that
    // finishes a chunk's last slab publishes the chunk's flag.
    constexpr int kParts = 4;
    constexpr int kPartRows = kBM / kParts;
    __shared__ int last_part;
    for (int item = blockIdx.x; item < t.chunks_per_rank * kParts; item += t.push_ctas) {
      const int chunk = item / kParts, part = item - chunk * kParts;
      const size_t row0 = size_t(chunk) * kBM + size_t(part) * kPartRows;
      const __nv_bfloat16* src = t.x_local + row0 * t.ldx;
      __nv_bfloat16* dst = t.gather_mc + half_off + (size_t(c.rank) * t.rows_per_rank + row0) * p.K;
      const int total = kPartRows * row_vecs;
      constexpr int kUnroll = 8;
      for (int i = threadIdx.x; i < total; i += kUnroll * blockDim.x) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int j = i + u * blockDim.x;
          if (j < total) {
            const int r = j / row_vecs, cv = j - r * row_vecs;
            v[u] = *reinterpret_cast<const uint4*>(src + size_t(r) * t.ldx + cv * 8);
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int j = i + u * blockDim.x;
          if (j < total) {
            const int r = j / row_vecs, cv = j - r * row_vecs;
            multimem_st16(dst + size_t(r) * p.K + cv * 8, v[u]);
          }
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t done = atomicAdd(t.counters + 1 + chunk, 1u);
        last_part = (done == uint32_t(kParts) - 1u);
        if (last_part) {
          t.counters[1 + chunk] = 0;
          __threadfence_system();
        }
      }
      __syncthreads();
      if (last_part && threadIdx.x < c.world)
        st_release_sys(c.flags[threadIdx.x] + (kTpChReady0 + chunk) * kMaxRanks + c.rank, q + 1u);
      __syncthreads();
    }
    return;
  }
  const int items = c.world * t.chunks_per_rank;
  for (int item = blockIdx.x; item < items; item += t.push_ctas) {
    const int d = item / t.chunks_per_rank;                      // 0 = own buffer, 1 = rank + 1, ...
    const int chunk = item - d * t.chunks_per_rank;
    const int peer = (c.rank + d) % c.world;
    const __nv_bfloat16* src = t.x_local + size_t(chunk) * kBM * t.ldx;
    __nv_bfloat16* dst = t.gather[peer] + half_off + (size_t(c.rank) * t.rows_per_rank + size_t(chunk) * kBM) * p.K;
    const int total = kBM * row_vecs;
    constexpr int kUnroll = 8;                 // 8 x 16 bytes per thread in flight: the loop is latency-bound
    for (int i = threadIdx.x; i < total; i += kUnroll * blockDim.x) {
      uint4 v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int j = i + u * blockDim.x;
        if (j < total) {
          const int r = j / row_vecs, cv = j - r * row_vecs;
          v[u] = *reinterpret_cast<const uint4*>(src + size_t(r) * t.ldx + cv * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int j = i + u * blockDim.x;
        if (j < total) {
          const int r = j / row_vecs, cv = j - r * row_vecs;
          *reinterpret_cast<uint4*>(dst + size_t(r) * p.K + cv * 8) = v[u];
        }
      }
    }
    __syncthreads();                           // one fence by the signalling thread covers the CTA's stores
    if (threadIdx.x == 0) __threadfence_system();
    if (threadIdx.x == 0) st_release_sys(c.flags[peer] + (kTpChReady0 + chunk) * kMaxRanks + c.rank, q + 1u);
  }
}

// mode 2, epilogue warps of a CTA that ran out of tiles: sum the W staged copies of this rank's rows.
__device__ void tp_reduce_rows(const GemmParams& p, const TpParams& t, const CommCtx& c, uint32_t q, int cta, int ncta,
                               int tid128, volatile uint32_t* abort_flag) {
  constexpr int kRowsPerItem = 8;
  const int items = t.rows_per_rank / kRowsPerItem;
  const int vec_per_row = p.N / 8;
  const __nv_bfloat16* base = t.stage[c.rank] + (long long)(q & 1u) * t.stage_half;
  const size_t slot = size_t(t.rows_per_rank) * p.N;
  int ready_chunk = -1;
  if (epi_any(*abort_flag != 0u)) return;      // another role of this CTA gave up: do not wait for flags
  for (int item = cta; item < items; item += ncta) {
    const int row0 = item * kRowsPerItem;
    const int chunk = row0 / kBM;
    if (chunk != ready_chunk) {
      bool failed = false;
      if (tid128 < c.world)
        failed = !tp_poll(c.flags[c.rank] + (kTpChReady0 + chunk) * kMaxRanks + tid128, q + 1u, c.st,
                          (41u << 16) | (uint32_t(chunk) << 4) | tid128);
      if (epi_any(failed)) {
        *abort_flag = 1u;
        return;
      }
      ready_chunk = chunk;
    }
    if (t.stage_mc != nullptr) {
      // every rank wrote its partial rows at the same offset of its own staging area: one reducing load through
      // the switch returns their sum. Several requests per thread are issued before the first result is used.
      const __nv_bfloat16* mc_rows = t.stage_mc + (long long)(q & 1u) * t.stage_half +
                                     size_t(c.rank) * t.rows_per_rank * p.N;
      const int total = kRowsPerItem * vec_per_row;
      constexpr int kPull = 8;                  // reducing loads in flight per thread
      for (int i0 = tid128; i0 < total; i0 += kPull * 128) {
        uint4 sum[kPull];
#pragma unroll
        for (int u = 0; u < kPull; ++u) {
          const int i = i0 + u * 128;
          if (i < total)
            sum[u] = multimem_ld_reduce16(mc_rows + size_t(row0 + i / vec_per_row) * p.N + (i % vec_per_row) * 8);
        }
#pragma unroll
        for (int u = 0; u < kPull; ++u) {
          const int i = i0 + u * 128;
          if (i < total) {
            const int r = row0 + i / vec_per_row;
            const int col = (i % vec_per_row) * 8;
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            accum_bf16x8(acc, sum[u], 1.f);
            if (t.rs_bias) accum_bf16x8(acc, __ldg(reinterpret_cast<const uint4*>(t.rs_bias + col)), 1.f);
            if (t.rs_residual)
              accum_bf16x8(acc, __ldg(reinterpret_cast<const uint4*>(t.rs_residual + size_t(r) * t.rs_ldr + col)), 1.f);
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
            o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
            *reinterpret_cast<uint4*>(t.out + size_t(r) * t.ldo + col) = o;
          }
        }
      }
      continue;
    }
    for (int i = tid128; i < kRowsPerItem * vec_per_row; i += 128) {
      const int r = row0 + i / vec_per_row;
      const int col = (i % vec_per_row) * 8;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      uint4 part[kMaxRanks];
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s)         // all loads first: eight 16-byte requests in flight per thread
        if (s < c.world) part[s] = __ldcg(reinterpret_cast<const uint4*>(base + s * slot + size_t(r) * p.N + col));
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s)
        if (s < c.world) accum_bf16x8(acc, part[s], 1.f);
      if (t.rs_bias) accum_bf16x8(acc, __ldg(reinterpret_cast<const uint4*>(t.rs_bias + col)), 1.f);
      if (t.rs_residual)
        accum_bf16x8(acc, __ldg(reinterpret_cast<const uint4*>(t.rs_residual + size_t(r) * t.rs_ldr + col)), 1.f);
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(t.out + size_t(r) * t.ldo + col) = o;
    }
  }
}

template <int B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
               const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
               const __grid_constant__ CUtensorMap tmAux, const GemmParams p, const TpParams t, const CommCtx c) {
  using L = TpSmem;
  constexpr int BN = kTpBN;
  constexpr int kStages = kTpStages;
  const uint32_t q = *t.seq;
  const int first_gemm_cta = (t.mode == 1) ? t.push_ctas : 0;

  if (int(blockIdx.x) < first_gemm_cta) {
    tp_push_rows(p, t, c, q);
  } else {
    extern __shared__ uint8_t smem_raw[];
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
    const int cta = int(blockIdx.x) - first_gemm_cta;
    const int ncta = int(gridDim.x) - first_gemm_cta;
    const int k_blocks = (p.K + kBK - 1) / kBK;
    const int units = p.m_tiles * p.n_tiles;
    const uint32_t* my_flags = c.flags[c.rank];

    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], 1);
      }
      for (int b = 0; b < 2; ++b) {
        mbar_init(&tmem_full[b], 1);
        mbar_init(&tmem_empty[b], 128);
      }
      *abort_flag = 0;
      fence_barrier_init();
    }
    if (warp == 1) {
      tmem_alloc(tmem_slot, 2 * BN);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        const CUtensorMap* tma = (t.mode == 1 && (q & 1u)) ? &tmA1 : &tmA0;
        tma_prefetch_desc(tma);
        tma_prefetch_desc(&tmB);
        int stage = 0;
        uint32_t phase = 0;
        uint32_t issued_mask = 0, issued_phase = 0;
        bool ok = true;
        for (int unit = cta; unit < units && ok; unit += ncta) {
          int tm, tn, owner, chunk;
          tp_unit_to_tile(p, t, c, unit, tm, tn, owner, chunk);
          if (t.mode == 1) {
            // the rows of this tile are pushed by `owner`; its chunk flag says they have landed
            if (!tp_poll(my_flags + (kTpChReady0 + chunk) * kMaxRanks + owner, q + 1u, p.st,
                         (42u << 16) | (uint32_t(chunk) << 4) | uint32_t(owner))) {
              *abort_flag = 1u;
              ok = false;
              break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");   // peer stores (generic proxy) before TMA reads
          }
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (3u << 16) | stage)) {
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * L::kStageBytes;
            uint8_t* sb = sa + L::kABytes;
            mbar_expect_tx(&full[stage], L::kStageBytes);
            tma_load_2d(sa, tma, &full[stage], kb * kBK, tm * kBM);
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmB, &full[stage], tn * BN + j * 64, kb * kBK);
            } else {
              tma_load_2d(sb, &tmB, &full[stage], kb * kBK, tn * BN);
            }
            issued_mask |= 1u << stage;
            issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
        }
        if (!ok || *abort_flag) {
          for (int s = 0; s < kStages; ++s) {
            if (issued_mask & (1u << s)) {
              const uint32_t par = (issued_phase >> s) & 1u;
              for (int i = 0; i < (1 << 20); ++i)
                if (mbar_try_wait(&full[s], par)) break;
            }
          }
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc_f16(kBM, BN, 0, B_MN, 1);
        int stage = 0;
        uint32_t phase = 0;
        int local = 0;
        bool ok = true;
        for (int unit = cta; unit < units && ok; unit += ncta, ++local) {
          const int buf = local & 1;
          const uint32_t acc_phase = (local >> 1) & 1;
          if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag, p.st, kTimeoutTmemEmpty, (3u << 16) | buf)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&full[stage], phase, abort_flag, p.st, kTimeoutSmemFull, (3u << 16) | stage)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
            const uint32_t sb = sa + L::kABytes;
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
              const uint64_t da = make_smem_desc_sw128(sa + kk * 32, 16, 1024);
              const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                                       : make_smem_desc_sw128(sb + kk * 32, 16, 1024);
              tc_mma_f16_ss(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
            tc_commit(&empty[stage]);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
          if (ok) tc_commit(&tmem_full[buf]);
        }
      }
    } else {
      // ---------------------------------------------------------------- epilogue (4 warps, 128 rows)
      const int quarter = warp & 3;
      const int tid128 = threadIdx.x - 64;
      const int row_in_tile = quarter * 32 + lane;
      uint8_t* my_stage = staging + quarter * 2 * 4096;
      const long long half_off = (long long)(q & 1u) * t.stage_half;
      int local = 0;
      int ring = 0;
      bool ok = true;
      if (t.mode == 2) {
        // the staging halves about to be written were last read by op q - 2 of their owners
        bool failed = false;
        if (tid128 < c.world) failed = !tp_poll(my_flags + kTpChDone * kMaxRanks + tid128, q - 1u, p.st, (43u << 16) | tid128);
        if (epi_any(failed)) {
          *abort_flag = 1u;
          ok = false;
        }
      }
      for (int unit = cta; unit < units && ok; unit += ncta, ++local) {
        int tm, tn, owner, chunk;
        tp_unit_to_tile(p, t, c, unit, tm, tn, owner, chunk);
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        bool failed = !mbar_wait(&tmem_full[buf], acc_phase, abort_flag, p.st, kTimeoutTmemFull, (3u << 16) | buf);
        if (t.mode == 2) failed = epi_any(failed);   // mode 2 has barriers below: leave the loop together
        if (failed) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int row = tm * kBM + row_in_tile;
        const int row0 = tm * kBM + quarter * 32;
        const int n0 = tn * BN;
        const bool gelu = (p.act == kActGelu);
        __nv_bfloat16* peer_rows = nullptr;
        if (t.mode == 2) {
          // multicast pull: the partial tile stays in this rank's own staging area at its global row; otherwise
          // it goes into the owner's slot of this rank
          peer_rows = (t.stage_mc != nullptr)
                          ? t.stage[c.rank] + half_off + (size_t(tm) * kBM + quarter * 32) * p.N
                          : t.stage[owner] + half_off +
                                (size_t(c.rank) * t.rows_per_rank + size_t(chunk) * kBM + quarter * 32) * p.N;
        }
#pragma unroll 1
        for (int s64 = 0; s64 < BN / 64; ++s64) {
          const int col0 = n0 + s64 * 64;
          if (col0 >= p.N) break;
          uint8_t* cbuf = my_stage + ((gelu || t.mode == 2) ? 0 : (ring & 1)) * 4096;
          uint8_t* abuf = my_stage + 4096;
          if (t.mode == 1) {
            if (lane == 0) {
              if (gelu) tma_store_wait_read<0>(); else tma_store_wait_read<1>();
            }
          }
          __syncwarp();
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN + s64 * 64 + h * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = col0 + h * 32 + g * 8;
              float v[8], pre[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) { v[i] = __uint_as_float(r[g * 8 + i]) * p.alpha; pre[i] = 0.f; }
              if (t.mode == 1 && row < p.M && col < p.N) epilogue_math8(p, row, col, v, min(8, p.N - col), false, pre);
              const int chunk16 = ((h * 4 + g) ^ (lane & 7)) << 4;
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(cbuf + lane * 128 + chunk16) = o;
              if (gelu) {
                uint4 a;
                a.x = pack_bf16x2(pre[0], pre[1]); a.y = pack_bf16x2(pre[2], pre[3]);
                a.z = pack_bf16x2(pre[4], pre[5]); a.w = pack_bf16x2(pre[6], pre[7]);
                *reinterpret_cast<uint4*>(abuf + lane * 128 + chunk16) = a;
              }
            }
          }
          if (t.mode == 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmC, cbuf, col0, row0);
              tma_store_commit();
              if (gelu) {
                tma_store_2d(&tmAux, abuf, col0, row0);
                tma_store_commit();
              }
            }
            ++ring;
          } else {
            // slab -> owner's staging rows: 8 lanes cover one 128-byte row segment, 4 rows per pass
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + (lane >> 3);
              const int ch = lane & 7;
              const uint4 o = *reinterpret_cast<const uint4*>(cbuf + rr * 128 + ((ch ^ (rr & 7)) << 4));
              *reinterpret_cast<uint4*>(peer_rows + size_t(rr) * p.N + col0 + ch * 8) = o;
            }
            __syncwarp();
          }
        }
        tc_fence_before();
        mbar_arrive(&tmem_empty[buf]);
        if (t.mode == 2) {
          // count the tile; the last tile of the 128-row chunk tells the owner that this rank's part is complete
          // (one system fence by the counting thread after the barrier covers the 128 threads' stores; a fence
          //  per thread costs a system-wide drain each)
          epi_bar_sync();
          if (tid128 == 0) {
            __threadfence_system();
            const uint32_t done = atomicAdd(t.counters + 1 + tm, 1u);
            if (done == uint32_t(p.n_tiles) - 1u) {
              t.counters[1 + tm] = 0;
              __threadfence_system();
              st_release_sys(c.flags[owner] + (kTpChReady0 + chunk) * kMaxRanks + c.rank, q + 1u);
            }
          }
        }
      }
      if (t.mode == 1 && lane == 0) tma_store_wait<0>();
      if (t.mode == 2 && ok) tp_reduce_rows(p, t, c, q, cta, ncta, tid128, abort_flag);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
      tc_fence_after();
      tmem_dealloc(tmem_base, 2 * BN);
    }
  }

  // ------------------------------------------------------------------ the last CTA closes the op
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t n = atomicAdd(t.counters, 1u);
    if (n == gridDim.x - 1) {
      t.counters[0] = 0;
      __threadfence_system();
      *t.seq = q + 1u;
      if (!t.hold_done) {
        for (int peer = 0; peer < c.world; ++peer)
          st_release_sys(c.flags[peer] + kTpChDone * kMaxRanks + c.rank, q + 1u);
      }
    }
  }
}

// Publishes "every op up to *seq is done" for a rank that ran an op with hold_done (it kept reading the gathered
// rows after the op, e.g. for a weight gradient). Must run before the rank's next fused op.
__global__ void tp_release_kernel(const CommCtx c, const uint32_t* seq) {
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + kTpChDone * kMaxRanks + c.rank, *seq);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int tp_operand_map(CUtensorMap* tm, const void* ptr, int mn_extent, int k_extent, int ld, int mn_major,
                          int box_mn) {
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  if (mn_major) {
    dims[0] = uint64_t(mn_extent); dims[1] = uint64_t(k_extent);
    box[0] = 64; box[1] = kBK;
  } else {
    dims[0] = uint64_t(k_extent); dims[1] = uint64_t(mn_extent);
    box[0] = kBK; box[1] = uint32_t(box_mn);
  }
  strides[0] = uint64_t(ld) * 2;
  return encode_tensor_map(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int B_MN>
static int tp_launch(const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b, const CUtensorMap& cm,
                     const CUtensorMap& aux, const GemmParams& p, const TpParams& t, const CommCtx& c, int grid,
                     cudaStream_t stream) {
  auto kern = tp_gemm_kernel<B_MN>;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TpSmem::kTotal));
      }))
    return e;
  kern<<<grid, kGemmThreads, TpSmem::kTotal, stream>>>(a0, a1, b, cm, aux, p, t, c);
  note_launches(1);
  return int(cudaGetLastError());
}

static void tp_base_params(GemmParams& p, int M, int N, int K) {
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.alpha = 1.f;
  p.splits = 1;
  p.m_tiles = M / kBM;
  p.n_tiles = (N + kTpBN - 1) / kTpBN;
  p.st = status_device_ptr();
}

}  // namespace idrak

using namespace idrak;

IDRAK_API int idrak_tp_counter_words(int M) { return 1 + M / kBM + 8; }
IDRAK_API int idrak_tp_max_rows_per_rank() { return kTpMaxChunks * kBM; }

// Y[M, N] = act(gather(X)[M, K] · W^T + bias), X row-sharded: this rank passes its rows [M / world, K].
//   gather_ptrs[p]  rank p's gather area, 2 * gather_half_elems bf16 (gather_half_elems >= M * K)
//   W               [N, K] (w_mn = 0) or stored [K, N] (w_mn = 1), local shard
//   seq, counters   device words shared by all fused ops of this rank (counters: idrak_tp_counter_words(M), zeroed)
//   gather_multicast  NVSwitch multicast address of the gather areas (one store reaches all ranks), or null
// Returns 0, a negative argument code, or a CUDA error.
IDRAK_API int idrak_tp_ag_gemm(const void* ctx, const void* x_local, int ldx, void* const* gather_ptrs,
                               long long gather_half_elems, const void* W, int ldw, int w_mn, void* C, int ldc, int M,
                               int N, int K, const void* bias, int act, void* aux, int ld_aux, void* seq,
                               void* counters, int push_ctas, int hold_done, void* gather_multicast, void* stream_) {
  CommCtx c;
  memcpy(&c, ctx, sizeof(c));
  if (M <= 0 || N <= 0 || K <= 0 || M % (c.world * kBM) || K % 8 || (ldx & 7) || (ldw & 7) || (ldc & 7)) return -2;
  const int rows = M / c.world;
  if (rows / kBM > kTpMaxChunks || gather_half_elems < (long long)M * K) return -3;
  if (act != kActNone && act != kActGelu) return -4;
  if (act == kActGelu && (aux == nullptr || (ld_aux & 7))) return -4;
  GemmParams p{};
  tp_base_params(p, M, N, K);
  p.C = C; p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.act = act;
  p.aux = static_cast<__nv_bfloat16*>(aux);
  p.ld_aux = ld_aux;
  p.tma_store = 1;
  TpParams t;
  memset(&t, 0, sizeof(t));
  t.mode = 1;
  t.rows_per_rank = rows;
  t.chunks_per_rank = rows / kBM;
  const int sms = sm_count();
  if (push_ctas <= 0) push_ctas = 16;
  if (push_ctas > sms / 4) push_ctas = sms / 4;
  t.push_ctas = push_ctas;
  t.hold_done = hold_done;
  t.seq = static_cast<uint32_t*>(seq);
  t.counters = static_cast<uint32_t*>(counters);
  t.x_local = static_cast<const __nv_bfloat16*>(x_local);
  t.ldx = ldx;
  for (int i = 0; i < c.world; ++i) t.gather[i] = static_cast<__nv_bfloat16*>(gather_ptrs[i]);
  t.gather_half = gather_half_elems;
  t.gather_mc = static_cast<__nv_bfloat16*>(gather_multicast);

  CUtensorMap a0, a1, b, cm, am;
  memset(&am, 0, sizeof(am));
  __nv_bfloat16* g = t.gather[c.rank];
  if (tp_operand_map(&a0, g, M, K, K, 0, kBM)) return -10;
  if (tp_operand_map(&a1, g + gather_half_elems, M, K, K, 0, kBM)) return -10;
  if (tp_operand_map(&b, W, N, K, ldw, w_mn, kTpBN)) return -12;
  {
    uint64_t dims[2] = {uint64_t(N), uint64_t(M)};
    uint32_t box[2] = {64, 32};
    uint64_t str_c[1] = {uint64_t(ldc) * 2};
    if (encode_tensor_map(&cm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, str_c, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return -13;
    if (act == kActGelu) {
      uint64_t str_a[1] = {uint64_t(ld_aux) * 2};
      if (encode_tensor_map(&am, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, aux, dims, str_a, box,
                            CU_TENSOR_MAP_SWIZZLE_128B))
        return -13;
    }
  }
  const int units = p.m_tiles * p.n_tiles;
  int gemm_ctas = sms - push_ctas;
  if (gemm_ctas > units) gemm_ctas = units;
  const int grid = push_ctas + gemm_ctas;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  return w_mn ? tp_launch<1>(a0, a1, b, cm, am, p, t, c, grid, s) : tp_launch<0>(a0, a1, b, cm, am, p, t, c, grid, s);
}

// After an idrak_tp_ag_gemm with hold_done: tell the peers that this rank has finished with the gathered rows.
IDRAK_API int idrak_tp_release(const void* ctx, const void* seq, void* stream_) {
  CommCtx c;
  memcpy(&c, ctx, sizeof(c));
  tp_release_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(c, static_cast<const uint32_t*>(seq));
  note_launches(1);
  return int(cudaGetLastError());
}

// out[M / world, N] = rows of this rank of sum over ranks (X_local[M, K] · W^T) (+ bias) (+ residual).
//   stage_ptrs[p]   rank p's staging area, 2 * stage_half_elems bf16 (stage_half_elems >= M * N)
//   W               [N, K] (w_mn = 0) or stored [K, N] (w_mn = 1), local shard over K
IDRAK_API int idrak_tp_gemm_rs(const void* ctx, const void* A, int lda, const void* W, int ldw, int w_mn,
                               void* const* stage_ptrs, long long stage_half_elems, void* out, int ldo, int M, int N,
                               int K, const void* bias, const void* residual, int ldr, void* seq, void* counters,
                               const void* stage_multicast, void* stream_) {
  CommCtx c;
  memcpy(&c, ctx, sizeof(c));
  if (M <= 0 || N <= 0 || K <= 0 || M % (c.world * kBM) || N % 64 || K % 8 || (lda & 7) || (ldw & 7) || (ldo & 7) ||
      (residual && (ldr & 7)))
    return -2;
  const int rows = M / c.world;
  if (rows / kBM > kTpMaxChunks || stage_half_elems < (long long)M * N) return -3;
  GemmParams p{};
  tp_base_params(p, M, N, K);
  TpParams t;
  memset(&t, 0, sizeof(t));
  t.mode = 2;
  t.rows_per_rank = rows;
  t.chunks_per_rank = rows / kBM;
  t.seq = static_cast<uint32_t*>(seq);
  t.counters = static_cast<uint32_t*>(counters);
  for (int i = 0; i < c.world; ++i) t.stage[i] = static_cast<__nv_bfloat16*>(stage_ptrs[i]);
  t.stage_half = stage_half_elems;
  t.stage_mc = static_cast<const __nv_bfloat16*>(stage_multicast);
  t.out = static_cast<__nv_bfloat16*>(out);
  t.ldo = ldo;
  t.rs_residual = static_cast<const __nv_bfloat16*>(residual);
  t.rs_ldr = ldr;
  t.rs_bias = static_cast<const __nv_bfloat16*>(bias);
  CUtensorMap a0, b, unused;
  memset(&unused, 0, sizeof(unused));
  if (tp_operand_map(&a0, A, M, K, lda, 0, kBM)) return -10;
  if (tp_operand_map(&b, W, N, K, ldw, w_mn, kTpBN)) return -12;
  const int units = p.m_tiles * p.n_tiles;
  const int sms = sm_count();
  const int grid = units < sms ? units : sms;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  return w_mn ? tp_launch<1>(a0, a0, b, unused, unused, p, t, c, grid, s)
              : tp_launch<0>(a0, a0, b, unused, unused, p, t, c, grid, s);
}
