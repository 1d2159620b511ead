// Dense bf16/fp16 GEMM for sm_100a: C[M,N] = epilogue(A · B), fp32 accumulation in TMEM.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer   (cp.async.bulk.tensor into a 128B-swizzled shared-memory ring)
//   warp 1      MMA issuer     (one thread issues tcgen05.mma; owns the TMEM allocation)
//   warps 2..9  epilogue       (tcgen05.ld the fp32 accumulator, fuse bias / GELU / GELU' / residual /
//                               accumulate, write bf16 or fp32; two groups of four warps, each group owning
//                               half of the tile's columns - see drain_accumulator in gemm_epilogue.cuh)
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps the
// main loop of tile i+1. Both operands may be K-major or MN-major in memory, which gives the four
// BLAS transposition cases without a transposed copy:
//   A K-major : A is [M,K] row-major          A MN-major : A is stored as [K,M] row-major
//   B K-major : B is [N,K] row-major          B MN-major : B is stored as [K,N] row-major
// (Linear forward = K/K, input gradient = K/MN, weight gradient = MN/MN.)
// Split-K writes fp32 partials to a workspace and a second kernel sums them in split order, so the
// result does not depend on scheduling.
//
// Covers the reference's tensor-core family gemm_tc_{nn,nt,tn,tt}_f32 and its bias / GELU / GELU-grad /
// residual epilogues (src/Idrak.Gpu/Cuda/PtxKernels.TensorCore.cs:24-29,80-144) and the host dispatch
// of CudaBackend.cs:1306-1471.
#include "gemm_epilogue.cuh"
#include <cstring>

namespace idrak {


template <int BN>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kStagingBytes = kDenseStagingBytes;   // per epilogue group: one 128-row x 128-byte slab
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;  // + alignment slack
};

// F8 = 1: both operands are e4m3 bytes, K-major; a 128-byte swizzle row then holds 128 elements of K, the MMA is
// kind::f8f6f4 (K = 32 per instruction, the same 32 bytes per step), everything else is unchanged.
//
// GROUPED (mixture-of-experts products over rows sorted by expert, segments padded to 128 rows):
//   1  every M tile belongs to one expert (p.tile_group): the B tile comes from that expert's slice of the stacked
//      weights; tiles beyond p.tiles_in_use (a device scalar) are not visited. Forward and input-gradient products.
//   2  one output per expert, C stacked [groups * M, N]; expert g contracts over its own rows only, blocks
//      [group_kb[g], group_kb[g + 1]) of K. An expert without rows gets zeros. Weight-gradient products.
//   3  not a grouped product: a second operand pair (tmA2, tmB2; p.extra_kb blocks of K) is contracted after the first
//      into the same accumulator, C = A B + A2 B2. This is how a low-rank adapter rides on its base projection: A2 is
//      the [M, r] product of the input with the adapter's down matrix, B2 the (scaled) up matrix, and the adapter costs
//      one more K block instead of a second pass over C. Columns of K beyond the operands' extent read as zeros.
template <int BN, int A_MN, int B_MN, int F8 = 0, int GROUPED = 0>
__global__ void __launch_bounds__(kDenseThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAux,
            const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
  using L = GemmSmem<BN>;
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + kStages * L::kStageBytes;        // 1024-byte aligned (stages are 16 KB multiples)
  uint8_t* bar_base = staging + L::kStagingBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kKB = F8 ? 2 * kBK : kBK;          // elements of K per shared-memory stage
  const int k_blocks_total = (p.K + kKB - 1) / kKB;
  const int kb_per_split = (k_blocks_total + p.splits - 1) / p.splits;
  const int m_tiles = (GROUPED == 1) ? min(p.m_tiles, *p.tiles_in_use) : p.m_tiles;
  const int units = (GROUPED == 2 ? p.groups : p.splits) * m_tiles * p.n_tiles;
  // unit -> tile (and expert / K range in the grouped modes); every role walks the same sequence
  auto tile_of = [&](int unit, int& tm, int& tn, int& split, int& group, int& kb0, int& kb1) {
    if (GROUPED == 2) {
      const int tiles = m_tiles * p.n_tiles;
      group = unit / tiles;
      unit_to_tile_n(m_tiles, p.n_tiles, unit - group * tiles, tm, tn, split);
      kb0 = p.group_kb[group];
      kb1 = p.group_kb[group + 1];
    } else {
      unit_to_tile_n(m_tiles, p.n_tiles, unit, tm, tn, split);
      group = (GROUPED == 1) ? p.tile_group[tm] : 0;
      kb0 = split * kb_per_split;
      kb1 = min(k_blocks_total, kb0 + kb_per_split);
      if (GROUPED == 3) kb1 += p.extra_kb;             // one pass over K (no split): the second pair follows the first
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 32 * kEpiWarps);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, issued_phase = 0;   // which stages have a copy in flight and on which parity
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
        int tm, tn, split, group, kb0, kb1;
        tile_of(unit, tm, tn, split, group, kb0, kb1);
        const int b_row = (GROUPED == 1) ? group * p.group_b_rows : 0;     // the expert's slice of the stacked B
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (1u << 16) | stage)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full[stage], L::kStageBytes);
          if (GROUPED == 3 && kb >= k_blocks_total) {
            const int k2 = (kb - k_blocks_total) * kKB;
            tma_load_2d(sa, &tmA2, &full[stage], k2, tm * kBM);
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmB2, &full[stage], tn * BN + j * 64, k2);
            } else {
              tma_load_2d(sb, &tmB2, &full[stage], k2, tn * BN);
            }
          } else if (A_MN) {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j) tma_load_2d(sa + j * 8192, &tmA, &full[stage], tm * kBM + j * 64, kb * kKB);
          } else {
            tma_load_2d(sa, &tmA, &full[stage], kb * kKB, tm * kBM);
          }
          if (GROUPED == 3 && kb >= k_blocks_total) {
            // loaded above from the second pair
          } else if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tmB, &full[stage], tn * BN + j * 64, kb * kKB + b_row);
          } else {
            tma_load_2d(sb, &tmB, &full[stage], kb * kKB, tn * BN + b_row);
          }
          issued_mask |= 1u << stage;
          issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok || *abort_flag) {
        // give up: let the copies already issued land before the CTA's shared memory goes away
        for (int s = 0; s < kStages; ++s) {
          if (issued_mask & (1u << s)) {
            uint32_t par = (issued_phase >> s) & 1u;
            for (int i = 0; i < (1 << 20); ++i)
              if (mbar_try_wait(&full[s], par)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = F8 ? make_idesc_e4m3(kBM, BN) : make_idesc_f16(kBM, BN, A_MN, B_MN, 1);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      unsigned long long t_acc = 0, t_ops = 0;
      const long long t_begin = p.prof ? clock64() : 0;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++local) {
        int tm, tn, split, group, kb0, kb1;
        tile_of(unit, tm, tn, split, group, kb0, kb1);
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        const long long c0 = p.prof ? clock64() : 0;
        if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag, p.st, kTimeoutTmemEmpty, (1u << 16) | buf)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (p.prof) t_acc += (unsigned long long)(clock64() - c0);
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          const long long c2 = p.prof ? clock64() : 0;
          if (!mbar_wait(&full[stage], phase, abort_flag, p.st, kTimeoutSmemFull, (1u << 16) | stage)) {
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
            if (F8) tc_mma_f8_ss(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
            else tc_mma_f16_ss(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty[stage]);   // releases the stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&tmem_full[buf]);
      }
      if (p.prof) {
        p.prof[blockIdx.x * 8 + 0] = (unsigned long long)(clock64() - t_begin);   // MMA warp's whole loop
        p.prof[blockIdx.x * 8 + 1] = t_acc;                                        // ... waiting for a free accumulator
        p.prof[blockIdx.x * 8 + 2] = t_ops;                                        // ... waiting for operand stages
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps, 128 rows)
    const int ewarp = warp - 2;
    int local = 0;
    bool ok = true;
    unsigned long long t_wait = 0, t_busy = 0;
    SideAhead ahead;
    ahead.ready = false;
    ahead.ring = 0;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++local) {
      int tm, tn, split, group, kb0, kb1;
      tile_of(unit, tm, tn, split, group, kb0, kb1);
      NextTile next{false, 0, 0};
      if (unit + int(gridDim.x) < units) {
        int nm, nn, ns, ng, n0, n1;
        tile_of(unit + gridDim.x, nm, nn, ns, ng, n0, n1);
        next = NextTile{true, ((GROUPED == 2 ? ng * m_tiles : 0) + nm) * kBM, nn * BN};
      }
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      const bool has_k = kb0 < kb1;              // a split past the end of K (or an expert without rows) gives zeros
      const int row_base = ((GROUPED == 2 ? group * m_tiles : 0) + tm) * kBM;    // stacked outputs: expert g's rows
      const long long c0 = p.prof ? clock64() : 0;
      if (!mbar_wait(&tmem_full[buf], acc_phase, abort_flag, p.st, kTimeoutTmemFull, (1u << 16) | buf)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const long long c1 = p.prof ? clock64() : 0;
      uint64_t* done = &tmem_empty[buf];
      drain_accumulator<BN, 1>(p, &tmC, &tmAux, tmem_base + buf * BN, ewarp, lane, row_base, tn * BN, split, has_k,
                            staging, ahead, next, [done]() {
                              tc_fence_before();
                              mbar_arrive(done);
                            });
      if (p.prof) {
        t_wait += (unsigned long long)(c1 - c0);
        t_busy += (unsigned long long)(clock64() - c1);
      }
    }
    if (p.tma_store && (ewarp & 3) == 2 && lane == 0) tma_store_wait<0>();   // the groups' leaders (lane quarter 0)
    if (p.prof && ewarp == 0 && lane == 0) {
      p.prof[blockIdx.x * 8 + 4] = t_wait;
      p.prof[blockIdx.x * 8 + 5] = t_busy;
      p.prof[blockIdx.x * 8 + 6] = (unsigned long long)local;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// Sum split-K partials in split order and run the fused epilogue. One thread per 8 columns.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const GemmParams p) {
  const int groups_per_row = (p.N + 7) / 8;
  const long long total = (long long)p.M * groups_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int row = int(i / groups_per_row);
    const int col = int(i - (long long)row * groups_per_row) * 8;
    const int nvalid = min(8, p.N - col);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float* w = p.workspace + (size_t(s) * p.M + row) * p.N + col;
      if (nvalid == 8 && ((reinterpret_cast<uintptr_t>(w) & 15) == 0)) {
        float4 a = reinterpret_cast<const float4*>(w)[0], b = reinterpret_cast<const float4*>(w)[1];
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
        v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
      } else {
        for (int j = 0; j < nvalid; ++j) v[j] += w[j];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= p.alpha;
    epilogue8(p, row, col, v, nvalid);
  }
}

// ---------------------------------------------------------------------------
// host launcher
// ---------------------------------------------------------------------------
template <int BN, int A_MN, int B_MN, int F8 = 0, int GROUPED = 0>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                       const CUtensorMap& tmAux, const GemmParams& p, int grid, cudaStream_t stream,
                       const CUtensorMap* tmA2 = nullptr, const CUtensorMap* tmB2 = nullptr) {
  using L = GemmSmem<BN>;
  auto kern = gemm_kernel<BN, A_MN, B_MN, F8, GROUPED>;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      }))
    return e;
  kern<<<grid, kDenseThreads, L::kTotal, stream>>>(tmA, tmB, tmC, tmAux, tmA2 ? *tmA2 : tmA, tmB2 ? *tmB2 : tmB, p);
  note_launches(1);
  return int(cudaGetLastError());
}

int pick_epi_mode(const GemmParams& p) {
  auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!p.tma_store || p.col_scale || p.row_scale_f) return kEpiGeneric;
  if (p.bias && !aligned(p.bias)) return kEpiGeneric;
  if (p.residual && (!aligned(p.residual) || (p.ldr & 7))) return kEpiGeneric;
  const bool b = p.bias != nullptr, r = p.residual != nullptr;
  if (p.act == kActNone) return b ? (r ? kEpiBiasRes : kEpiBias) : (r ? kEpiRes : kEpiPlain);
  if (p.act == kActGelu && !r) return b ? kEpiBiasGelu : kEpiGelu;
  if (p.act == kActGeluGrad && !b && !r && aligned(p.aux) && (p.ld_aux & 7) == 0) return kEpiGeluGrad;
  if (p.act == kActGeluD && !r) return b ? kEpiBiasGeluD : kEpiGeluD;
  if (p.act == kActMulAux && !b && !r && aligned(p.aux) && (p.ld_aux & 7) == 0) return kEpiMulAux;
  return kEpiGeneric;
}

// Role timers: with a buffer set, every dense GEMM CTA writes eight cycle counts at [blockIdx.x * 8]:
//   0 MMA warp, whole tile loop   1 of that, waiting for a drained accumulator   2 of that, waiting for operands
//   4 first epilogue warp waiting for a finished accumulator   5 the same warp draining   6 tiles this CTA ran
// (3 and 7 unused). They say which of the three roles bounds a shape. The buffer must hold 8 words per SM.
static std::atomic<unsigned long long*> g_role_timers{nullptr};
unsigned long long* role_timer_buffer() { return g_role_timers.load(std::memory_order_relaxed); }

static int make_operand_map(CUtensorMap* tm, const void* ptr, int mn_extent, int k_extent, int ld, int mn_major,
                            int box_mn, int fp16) {
  // K-major : memory [mn_extent rows][k_extent contiguous], row stride ld   -> box {64 k, box_mn rows}
  // MN-major: memory [k_extent rows][mn_extent contiguous], row stride ld   -> box {64 mn, 64 k rows}
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  if (mn_major) {
    dims[0] = uint64_t(mn_extent);
    dims[1] = uint64_t(k_extent);
    box[0] = 64;
    box[1] = kBK;
  } else {
    dims[0] = uint64_t(k_extent);
    dims[1] = uint64_t(mn_extent);
    box[0] = kBK;
    box[1] = uint32_t(box_mn);
  }
  strides[0] = uint64_t(ld) * 2;
  return encode_tensor_map(tm, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           const_cast<void*>(ptr), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace idrak

using namespace idrak;

// Switch the role timers on (a device buffer of 8 * SM-count 64-bit words) or off (null).
IDRAK_API void idrak_gemm_role_timers(void* device_buffer) {
  g_role_timers.store(static_cast<unsigned long long*>(device_buffer), std::memory_order_relaxed);
}

// Number of fp32 workspace elements a call with these sizes needs (0 when it will not split K).
IDRAK_API long long idrak_gemm_workspace_elems(int M, int N, int K, int splits) {
  if (splits <= 1) return 0;
  return (long long)splits * M * N;
}

// Pick a split-K factor so a small output still fills the machine. Deterministic in (M, N, K, sms).
IDRAK_API int idrak_gemm_pick_splits(int M, int N, int K, int bn) {
  const int sms = sm_count();
  const int tiles = ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
  const int kblocks = (K + kBK - 1) / kBK;
  if (tiles * 2 > sms || kblocks < 16) return 1;
  int s = sms / tiles;
  s = max(1, min(s, kblocks / 8));
  return min(s, 16);
}

// C = epilogue(alpha * op(A) op(B)).
//   a_mn = 0: A is [M,K] row-major (lda >= K); a_mn = 1: A is stored [K,M] row-major (lda >= M)
//   b_mn = 0: B is [N,K] row-major (ldb >= K); b_mn = 1: B is stored [K,N] row-major (ldb >= N)
// Leading dimensions are in elements and must be multiples of 8 for A and B (TMA strides are 16-byte
// multiples). C, aux and residual may have any leading dimension; unaligned rows take a scalar path.
// Returns 0, a cudaError, or a negative argument error.
IDRAK_API int idrak_gemm_bf16(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, void* C, int ldc,
                              int c_fp32, int M, int N, int K, const void* bias, const void* residual, int ldr,
                              int act, void* aux, int ld_aux, int beta, float alpha, int splits, float* workspace,
                              int fp16, void* stream_) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (act != kActNone && aux == nullptr) return -4;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int bn = (N <= 128) ? 128 : 256;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.act = act;
  p.aux = static_cast<__nv_bfloat16*>(aux);
  p.ld_aux = ld_aux;
  p.beta = beta;
  p.alpha = alpha;
  p.splits = (splits > 1 && workspace) ? splits : 1;
  {
    // every split must own at least one k-block
    const int kblocks = (K + kBK - 1) / kBK;
    if (p.splits > kblocks) p.splits = kblocks;
    const int per = (kblocks + p.splits - 1) / p.splits;
    p.splits = (kblocks + per - 1) / per;
  }
  p.workspace = workspace;
  p.m_tiles = (M + kBM - 1) / kBM;
  p.n_tiles = (N + bn - 1) / bn;
  p.st = status_device_ptr();
  p.col_scale = nullptr;

  CUtensorMap tmA, tmB;
  int e = make_operand_map(&tmA, A, M, K, lda, a_mn, kBM, fp16);
  if (e) return -10 - (e > 0 ? 0 : 1);
  e = make_operand_map(&tmB, B, N, K, ldb, b_mn, bn, fp16);
  if (e) return -12;

  // Output through TMA when the layout allows: bf16, no accumulate, 16-byte aligned rows.
  CUtensorMap tmC, tmAux;
  memset(&tmC, 0, sizeof(tmC));
  memset(&tmAux, 0, sizeof(tmAux));
  p.tma_store = 0;
  if (!c_fp32 && !beta && p.splits == 1 && (ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
      ((act != kActGelu && act != kActGeluD) || ((ld_aux % 8) == 0 && (reinterpret_cast<uintptr_t>(aux) & 15) == 0))) {
    uint64_t dims[2] = {uint64_t(N), uint64_t(M)};
    uint32_t box[2] = {64, 128};
    uint64_t str_c[1] = {uint64_t(ldc) * 2};
    int ok = encode_tensor_map(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, str_c, box,
                               CU_TENSOR_MAP_SWIZZLE_128B) == 0;
    if (ok && (act == kActGelu || act == kActGeluD)) {
      uint64_t str_a[1] = {uint64_t(ld_aux) * 2};
      ok = encode_tensor_map(&tmAux, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, aux, dims, str_a, box,
                             CU_TENSOR_MAP_SWIZZLE_128B) == 0;
    }
    p.tma_store = ok ? 1 : 0;
  }
  p.epi_mode = pick_epi_mode(p);
  p.prof = role_timer_buffer();

  // large one-pass products go to CTA pairs (256 x 256 tiles, cta_group::2)
  if (bn == 256 && gemm_pair_wanted(M, N, K, p.splits))
    return gemm_pair_launch(A, lda, a_mn, B, ldb, b_mn, tmC, tmAux, p, fp16, stream);

  const int units = p.m_tiles * p.n_tiles * p.splits;
  const int grid = min(units, sm_count());
  int rc;
#define IDRAK_GEMM_CASE(BN_, AM_, BM_) rc = launch_gemm<BN_, AM_, BM_>(tmA, tmB, tmC, tmAux, p, grid, stream)
  if (bn == 256) {
    if (!a_mn && !b_mn) IDRAK_GEMM_CASE(256, 0, 0);
    else if (!a_mn && b_mn) IDRAK_GEMM_CASE(256, 0, 1);
    else if (a_mn && !b_mn) IDRAK_GEMM_CASE(256, 1, 0);
    else IDRAK_GEMM_CASE(256, 1, 1);
  } else {
    if (!a_mn && !b_mn) IDRAK_GEMM_CASE(128, 0, 0);
    else if (!a_mn && b_mn) IDRAK_GEMM_CASE(128, 0, 1);
    else if (a_mn && !b_mn) IDRAK_GEMM_CASE(128, 1, 0);
    else IDRAK_GEMM_CASE(128, 1, 1);
  }
#undef IDRAK_GEMM_CASE
  if (rc) return rc;
  if (p.splits > 1) {
    const long long groups = (long long)M * ((N + 7) / 8);
    long long want = (groups + 255) / 256, cap = (long long)sm_count() * 8;
    int blocks = int(want < cap ? want : cap);
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p);
    note_launches(1);
    rc = int(cudaGetLastError());
  }
  return rc;
}

// C (bf16) = A op(B) + A2 op(B2) (+ bias) (+ residual): a product with a low-rank term contracted into the same
// accumulator. A [M, K] and A2 [M, K2] are row-major; B and B2 share one layout: [N, K] / [N, K2] (b_mn = 0) or stored
// [K, N] / [K2, N] (b_mn = 1). K2 is the adapter rank (or the ranks of several adapters side by side): any multiple
// of 8 up to 256; the tail of its last 64-element block reads as zeros. Leading dimensions are multiples of 8.
// Covers the reference's gemm_tc_{nn,nt}_lr_f32 family (src/Idrak.Gpu/Cuda/PtxKernels.TensorCore.cs:118-126): the
// adapter as one more k step of the base product.
IDRAK_API int idrak_gemm_lowrank(const void* A, int lda, const void* B, int ldb, int b_mn, const void* A2, int lda2,
                                 const void* B2, int ldb2, void* C, int ldc, int M, int N, int K, int K2,
                                 const void* bias, const void* residual, int ldr, void* stream_) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K2 <= 0 || K2 > 256 || (K2 & 7)) return -2;
  if ((lda & 7) || (ldb & 7) || (lda2 & 7) || (ldb2 & 7)) return -2;
  for (const void* q : {A, B, A2, B2})
    if (reinterpret_cast<uintptr_t>(q) & 15) return -3;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int bn = (N <= 128) ? 128 : 256;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.c_fp32 = 0;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.act = kActNone;
  p.alpha = 1.f;
  p.splits = 1;
  p.m_tiles = (M + kBM - 1) / kBM;
  p.n_tiles = (N + bn - 1) / bn;
  p.st = status_device_ptr();
  p.extra_kb = (K2 + kBK - 1) / kBK;
  CUtensorMap tmA, tmB, tmA2, tmB2, tmC, tmAux;
  if (make_operand_map(&tmA, A, M, K, lda, 0, kBM, 0)) return -11;
  if (make_operand_map(&tmB, B, N, K, ldb, b_mn, bn, 0)) return -12;
  if (make_operand_map(&tmA2, A2, M, K2, lda2, 0, kBM, 0)) return -13;
  if (make_operand_map(&tmB2, B2, N, K2, ldb2, b_mn, bn, 0)) return -14;
  memset(&tmC, 0, sizeof(tmC));
  memset(&tmAux, 0, sizeof(tmAux));
  p.tma_store = 0;
  if ((ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
    uint64_t dims[2] = {uint64_t(N), uint64_t(M)};
    uint32_t box[2] = {64, 128};
    uint64_t str_c[1] = {uint64_t(ldc) * 2};
    p.tma_store = encode_tensor_map(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, str_c, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B) == 0;
  }
  p.epi_mode = pick_epi_mode(p);
  p.prof = nullptr;
  const int grid = min(p.m_tiles * p.n_tiles, sm_count());
  if (bn == 256)
    return b_mn ? launch_gemm<256, 0, 1, 0, 3>(tmA, tmB, tmC, tmAux, p, grid, stream, &tmA2, &tmB2)
                : launch_gemm<256, 0, 0, 0, 3>(tmA, tmB, tmC, tmAux, p, grid, stream, &tmA2, &tmB2);
  return b_mn ? launch_gemm<128, 0, 1, 0, 3>(tmA, tmB, tmC, tmAux, p, grid, stream, &tmA2, &tmB2)
              : launch_gemm<128, 0, 0, 0, 3>(tmA, tmB, tmC, tmAux, p, grid, stream, &tmA2, &tmB2);
}

// C[M, N] (bf16) = (A B^T) * row_scale[m] * col_scale[n] (+ bias) with A [M, K] and B [N, K] e4m3 bytes, K-major
// (lda, ldb in bytes, multiples of 16; K a multiple of 16). fp32 accumulation on the kind::f8f6f4 tensor path.
// Covers the reference's gemm8_e4m3_f32 with per-row A scales and per-column B scales applied in the epilogue
// (src/Idrak.Gpu/Cuda/PtxKernels.EightBit.cs:17-23).
IDRAK_API int idrak_gemm_fp8(const void* A, int lda, const void* B, int ldb, void* C, int ldc, int M, int N, int K,
                             const float* row_scale, const float* col_scale, const void* bias, void* stream_) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 15) || (ldb & 15) || (K & 15)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (!row_scale || !col_scale) return -4;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int bn = (N <= 128) ? 128 : 256;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.c_fp32 = 0;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.act = kActNone;
  p.alpha = 1.f;
  p.splits = 1;
  p.m_tiles = (M + kBM - 1) / kBM;
  p.n_tiles = (N + bn - 1) / bn;
  p.st = status_device_ptr();
  p.row_scale_f = row_scale;
  p.col_scale_f = col_scale;
  auto byte_map = [](CUtensorMap* tm, const void* ptr, int rows, int k, int ld, int box_rows) {
    uint64_t dims[2] = {uint64_t(k), uint64_t(rows)};
    uint64_t strides[1] = {uint64_t(ld)};
    uint32_t box[2] = {128, uint32_t(box_rows)};
    return encode_tensor_map(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B);
  };
  CUtensorMap tmA, tmB, tmC, tmAux;
  if (byte_map(&tmA, A, M, K, lda, kBM)) return -11;
  if (byte_map(&tmB, B, N, K, ldb, bn)) return -12;
  memset(&tmC, 0, sizeof(tmC));
  memset(&tmAux, 0, sizeof(tmAux));
  p.tma_store = 0;
  if ((ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
    uint64_t dims[2] = {uint64_t(N), uint64_t(M)};
    uint32_t box[2] = {64, 128};
    uint64_t str_c[1] = {uint64_t(ldc) * 2};
    p.tma_store = encode_tensor_map(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, str_c, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B) == 0;
  }
  p.epi_mode = kEpiGeneric;
  p.prof = nullptr;
  const int units = p.m_tiles * p.n_tiles;
  const int grid = min(units, sm_count());
  if (bn == 256) return launch_gemm<256, 0, 0, 1>(tmA, tmB, tmC, tmAux, p, grid, stream);
  return launch_gemm<128, 0, 0, 1>(tmA, tmB, tmC, tmAux, p, grid, stream);
}

// ---------------------------------------------------------------------------
// grouped products for mixture-of-experts layers (rows sorted by expert, segments padded to 128 rows)
// ---------------------------------------------------------------------------
namespace {

int grouped_store_map(CUtensorMap* tm, void* C, int rows, int N, int ldc) {
  uint64_t dims[2] = {uint64_t(N), uint64_t(rows)};
  uint32_t box[2] = {64, 128};
  uint64_t str_c[1] = {uint64_t(ldc) * 2};
  return encode_tensor_map(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, str_c, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

// C[cap, N] = A[cap, K] x B_e, expert e = tile_group[row / 128], for the first *tiles_in_use row tiles.
//   b_mn = 0: B stacked [E * N, K] (the nn.Linear layout per expert): C = A B_e^T        (forward)
//   b_mn = 1: B stacked [E * K, N]:                                   C = A B_e          (input gradient)
// K must be a multiple of 64 (a K block must not run into the next expert's rows), lda / ldb / ldc multiples of 8.
// Reference: expert_matmul (src/Idrak.Gpu/Cuda/PtxKernels.Routing.cs:30-35), which loops over experts on the host.
IDRAK_API int idrak_gemm_grouped_rows(const void* A, int lda, const void* B, int ldb, int b_mn, void* C, int ldc,
                                      int cap, int N, int K, int experts, const int* tile_group,
                                      const int* tiles_in_use, void* stream_) {
  if (cap <= 0 || N <= 0 || K <= 0) return 0;
  if ((cap % kBM) || (K % kBK) || (lda & 7) || (ldb & 7) || (ldc & 7) || (N & 7)) return -2;
  if (!tile_group || !tiles_in_use) return -3;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int bn = (N <= 128) ? 128 : 256;
  GemmParams p{};
  p.M = cap; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.alpha = 1.f;
  p.splits = 1;
  p.m_tiles = cap / kBM;
  p.n_tiles = (N + bn - 1) / bn;
  p.st = status_device_ptr();
  p.tile_group = tile_group;
  p.tiles_in_use = tiles_in_use;
  p.group_b_rows = b_mn ? K : N;
  CUtensorMap tmA, tmB, tmC, tmAux;
  memset(&tmAux, 0, sizeof(tmAux));
  if (make_operand_map(&tmA, A, cap, K, lda, 0, kBM, 0)) return -10;
  // the stacked weights as one 2-D array: [E * N rows, K] or [E * K rows, N]
  if (b_mn ? make_operand_map(&tmB, B, N, experts * K, ldb, 1, bn, 0)
           : make_operand_map(&tmB, B, experts * N, K, ldb, 0, bn, 0))
    return -12;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || grouped_store_map(&tmC, C, cap, N, ldc)) return -13;
  p.tma_store = 1;
  p.epi_mode = pick_epi_mode(p);
  p.prof = nullptr;
  const int grid = min(p.m_tiles * p.n_tiles, sm_count());
  if (bn == 256)
    return b_mn ? launch_gemm<256, 0, 1, 0, 1>(tmA, tmB, tmC, tmAux, p, grid, stream)
                : launch_gemm<256, 0, 0, 0, 1>(tmA, tmB, tmC, tmAux, p, grid, stream);
  return b_mn ? launch_gemm<128, 0, 1, 0, 1>(tmA, tmB, tmC, tmAux, p, grid, stream)
              : launch_gemm<128, 0, 0, 0, 1>(tmA, tmB, tmC, tmAux, p, grid, stream);
}

// dW_e [M, N] = A[rows of e, M]^T x B[rows of e, N] for every expert e, written to C stacked [E * M, N] (bf16, or
// fp32 with `c_fp32`; `beta` adds to what C holds). Rows of expert e are blocks [group_kb[e], group_kb[e + 1]) of
// 64 rows of A and B; padding rows inside a segment must be zero. M must be a multiple of 128.
IDRAK_API int idrak_gemm_grouped_k(const void* A, int lda, const void* B, int ldb, void* C, int ldc, int c_fp32,
                                   int beta, int cap, int M, int N, int experts, const int* group_kb, void* stream_) {
  if (cap <= 0 || M <= 0 || N <= 0 || experts <= 0) return 0;
  if ((M % kBM) || (cap % kBK) || (lda & 7) || (ldb & 7) || (N & 7)) return -2;
  if (!group_kb) return -3;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int bn = (N <= 128) ? 128 : 256;
  GemmParams p{};
  p.M = experts * M; p.N = N; p.K = cap;
  p.C = C; p.ldc = ldc; p.c_fp32 = c_fp32;
  p.beta = beta;
  p.alpha = 1.f;
  p.splits = 1;
  p.m_tiles = M / kBM;
  p.n_tiles = (N + bn - 1) / bn;
  p.st = status_device_ptr();
  p.group_kb = group_kb;
  p.groups = experts;
  CUtensorMap tmA, tmB, tmC, tmAux;
  memset(&tmC, 0, sizeof(tmC));
  memset(&tmAux, 0, sizeof(tmAux));
  if (make_operand_map(&tmA, A, M, cap, lda, 1, kBM, 0)) return -10;
  if (make_operand_map(&tmB, B, N, cap, ldb, 1, bn, 0)) return -12;
  p.tma_store = 0;
  if (!c_fp32 && !beta && (ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0)
    p.tma_store = grouped_store_map(&tmC, C, experts * M, N, ldc) == 0 ? 1 : 0;
  p.epi_mode = pick_epi_mode(p);
  p.prof = nullptr;
  const int grid = min(experts * p.m_tiles * p.n_tiles, sm_count());
  if (bn == 256) return launch_gemm<256, 1, 1, 0, 2>(tmA, tmB, tmC, tmAux, p, grid, stream);
  return launch_gemm<128, 1, 1, 0, 2>(tmA, tmB, tmC, tmAux, p, grid, stream);
}
