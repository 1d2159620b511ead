// Few-row products for decoding: C[M, N] = X[M, K] W[N, K]^T with M <= 64 tokens, bound by streaming W once.
//
// The product is computed transposed, so the weights fill the 128-row side of the tensor-core tile and the tokens the
// narrow side: D[128 features, NT tokens] += W_tile[128, 64] X_tile[NT, 64]^T per K block (tcgen05.mma M = 128,
// N = NT in {16, 32, 64}, fp32 accumulator in 64 TMEM columns). One tile of 128 output features belongs to a CLUSTER
// of 1, 2, 4 or 8 CTAs that split K between them, which is what fills the machine when N / 128 is below the SM count
// (a 4096-wide projection is 32 tiles). Each CTA:
//   warp 0      TMA producer: its K range of the W tile (16 KB per block) and of X (NT x 64) through a 4-stage ring
//   warp 1      MMA issuer
//   warps 2..5  meanwhile sum the squares of this CTA's K range of X (only when the RMS norm is folded in), then move
//               the accumulator into shared memory
// then the cluster meets, CTA r sums rows [r S, (r + 1) S) (S = 128 / cluster size) of all partial tiles through
// distributed shared memory in rank order - deterministic, no second kernel, no fp32 workspace in HBM - and runs the
// epilogue on its slice:
//   norm fold   y *= rsqrt(mean_k x^2 + eps): with the norm weight multiplied into W's columns beforehand this is
//               RMSNorm(x) W^T without a norm launch or a normalised copy of x
//   bias, residual add
//   gated       W holds [gate rows; up rows]; a tile pairs 64 gate features with their 64 up features (each CTA's
//               slice holds matching halves) and writes act(gate) * up: no [M, 2 ff] round trip, no activation launch
// Shared memory is 98 KB per CTA so two CTAs share an SM (192 KB of loads in flight per SM).
//
// Every mbarrier wait is bounded (status word + abort flag); every thread reaches both cluster barriers whatever
// happened before, so no CTA leaves while a peer still reads its shared memory.
//
// Reference counterparts: the few-row GEMV family with fused epilogues (src/Idrak.Gpu/Cuda/PtxKernels.Quantized.cs:13,
// 454-495: *_gemv_multi, _multi_act, _addnorm, _normaddnorm) and PtxKernels.Rows.cs:2047-2060.
#include "common.cuh"
#include <cstdlib>

namespace idrak {

constexpr int kSkFeat = 128;     // output features per tile (MMA M)
constexpr int kSkBK = 64;        // K elements per stage
constexpr int kSkStages = 4;
constexpr int kSkThreads = 192;

struct SkinnyParams {
  const __nv_bfloat16* X;        // [M, ldx]
  int ldx;
  __nv_bfloat16* C;              // [M, ldc]
  int ldc;
  const __nv_bfloat16* bias;     // [N] or null
  const __nv_bfloat16* residual; // [M, ldr] or null
  int ldr;
  int M, N, K;                   // N = output features (gated: ff)
  int gate_kind;                 // -1: plain; else 0 silu, 1 gelu (tanh), 2 relu
  int up_offset;                 // gated: row of W where the up rows start
  float norm_eps;                // >= 0: multiply row m by rsqrt(sum_k x[m,k]^2 / K + eps)
  int csize;                     // CTAs per cluster = K splits
  Status* st;
};

template <int NT>
struct SkinnySmem {
  static constexpr int kW = kSkFeat * kSkBK * 2;          // 16 KB
  static constexpr int kX = NT * kSkBK * 2;
  static constexpr int kStage = kW + 64 * kSkBK * 2;      // X slot sized for 64 tokens so stages stay 1024-aligned
  // after the main loop the drained stages are reused: the partial tile [NT][128] fp32 (read by the whole cluster)
  // and this CTA's reduced slice [NT][S] fp32, 32 KB each at most
  static constexpr int kPart = 0;
  static constexpr int kRed = 32768;
  static constexpr int kSs = kSkStages * kStage;           // ss_part[64], ss[64]
  static constexpr int kBar = kSs + 64 * 4 * 2;
  static constexpr int kTotal = kBar + 256 + 1024;
};

__device__ __forceinline__ uint32_t sk_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t sk_map_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ float sk_ld_cluster(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 sk_ld_cluster4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sk_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ float sk_gate(float g, int kind) {
  if (kind == 0) return g / (1.f + __expf(-g));
  if (kind == 1) return gelu_tanh(g);
  return fmaxf(g, 0.f);
}

template <int NT>
__global__ void __launch_bounds__(kSkThreads, 2)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const SkinnyParams p) {
  using L = SkinnySmem<NT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* part = reinterpret_cast<float*>(smem + L::kPart);
  float* red = reinterpret_cast<float*>(smem + L::kRed);
  float* ss_part = reinterpret_cast<float*>(smem + L::kSs);
  float* ss = ss_part + 64;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* empty = full + kSkStages;
  uint64_t* acc_full = empty + kSkStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int csize = p.csize;
  const int rank = int(sk_cluster_rank());
  const int tile = blockIdx.x / csize;
  const int S = kSkFeat / csize;                       // tile rows this CTA reduces and finishes
  const bool gated = p.gate_kind >= 0;
  const int kblocks = (p.K + kSkBK - 1) / kSkBK;
  const int per = (kblocks + csize - 1) / csize;
  const int kb0 = min(kblocks, rank * per), kb1 = min(kblocks, kb0 + per);

  pdl_launch_dependents();
  // one stage of operands: the weight tile (or the gate and up slices of a gated pair) and the token rows
  auto issue = [&](int kb, int stage) {
    uint8_t* sw = smem + stage * L::kStage;
    uint8_t* sx = sw + L::kW;
    mbar_expect_tx(&full[stage], L::kW + L::kX);
    if (!gated) {
      tma_load_2d(sw, &tmW, &full[stage], kb * kSkBK, tile * kSkFeat);
    } else {
      // slice r of the tile: S / 2 gate rows then the S / 2 up rows of the same features
      const int half = S / 2;
      for (int r = 0; r < csize; ++r) {
        const int f = tile * 64 + r * half;
        tma_load_2d(sw + (r * S) * 128, &tmW, &full[stage], kb * kSkBK, f);
        tma_load_2d(sw + (r * S + half) * 128, &tmW, &full[stage], kb * kSkBK, p.up_offset + f);
      }
    }
    tma_load_2d(sx, &tmX, &full[stage], kb * kSkBK, 0);
  };
  const int first = min(kSkStages, kb1 - kb0);          // stages filled before the CTA-wide sync (all are free then)
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSkStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
    pdl_wait();                                          // the kernels before this one have written the token rows
    for (int i = 0; i < first; ++i) issue(kb0 + i, i);   // in flight while tensor memory is allocated below
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();                                            // every thread that reads global memory (rows, bias, residual)
  const uint32_t tmem_acc = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      int stage = first % kSkStages;
      uint32_t phase = first == kSkStages ? 1u : 0u;
      uint32_t issued_mask = (1u << first) - 1u, issued_phase = 0;
      for (int kb = kb0 + first; kb < kb1 && ok; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (7u << 16) | stage)) {
          ok = false;
          break;
        }
        issue(kb, stage);
        issued_mask |= 1u << stage;
        issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
        if (++stage == kSkStages) { stage = 0; phase ^= 1; }
      }
      if (!ok || *abort_flag) {
        for (int s = 0; s < kSkStages; ++s) {
          if (issued_mask & (1u << s)) {
            const uint32_t par = (issued_phase >> s) & 1u;
            for (int i = 0; i < (1 << 20); ++i)
              if (mbar_try_wait(&full[s], par)) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kSkFeat, NT, 0, 0, 1);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag, p.st, kTimeoutSmemFull, (7u << 16) | (8 + stage))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sw = smem_u32(smem + stage * L::kStage);
        const uint32_t sx = sw + L::kW;
#pragma unroll
        for (int kk = 0; kk < kSkBK / 16; ++kk) {
          const uint64_t da = make_smem_desc_sw128(sw + kk * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sx + kk * 32, 16, 1024);
          tc_mma_f16_ss(tmem_acc, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&empty[stage]);
        if (++stage == kSkStages) { stage = 0; phase ^= 1; }
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps, part one
    const int ew = warp - 2;
    if (p.norm_eps >= 0.f) {
      // sum of squares of this CTA's K range, one warp per token row (rows ew, ew + 4, ...)
      const int k_lo = kb0 * kSkBK, k_hi = min(p.K, kb1 * kSkBK);
      for (int m = ew; m < NT; m += 4) {
        float acc = 0.f;
        if (m < p.M) {
          const __nv_bfloat16* row = p.X + size_t(m) * p.ldx;
          for (int k = k_lo + lane * 8; k < k_hi; k += 256) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + k));
            float2 f;
            f = unpack_bf16x2(v.x); acc += f.x * f.x + f.y * f.y;
            f = unpack_bf16x2(v.y); acc += f.x * f.x + f.y * f.y;
            f = unpack_bf16x2(v.z); acc += f.x * f.x + f.y * f.y;
            f = unpack_bf16x2(v.w); acc += f.x * f.x + f.y * f.y;
          }
        }
        acc = warp_sum(acc);
        if (lane == 0) ss_part[m] = acc;
      }
    }
    const bool have = kb1 > kb0;
    if (have) ok = mbar_wait(acc_full, 0, abort_flag, p.st, kTimeoutTmemFull, (7u << 16) | 32);
    tc_fence_after();
    const int q = warp & 3;                            // the TMEM lane quarter this warp may read
    const int f = q * 32 + lane;                       // tile row = accumulator lane
    if (have && ok) {
#pragma unroll
      for (int c = 0; c < NT / 16; ++c) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(tmem_acc + (uint32_t(q * 32) << 16) + c * 16, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) part[(c * 16 + i) * kSkFeat + f] = __uint_as_float(v[i]);
      }
    } else {
      for (int m = 0; m < NT; ++m) part[m * kSkFeat + f] = 0.f;      // no K blocks here (or gave up): contributes zeros
    }
  }

  // every thread of every CTA of the cluster: partial tiles (and partial sums of squares) are complete and visible
  tc_fence_before();
  __syncwarp();
  sk_cluster_sync();

  if (warp >= 2) {
    const int t = threadIdx.x - 64;                   // 0 .. 127
    const uint32_t part_addr = smem_u32(part), ssp_addr = smem_u32(ss_part);
    if (p.norm_eps >= 0.f && t < NT) {
      float a = 0.f;
      for (int r = 0; r < csize; ++r) a += sk_ld_cluster(sk_map_rank(ssp_addr + t * 4, r));
      ss[t] = rsqrtf(a / float(p.K) + p.norm_eps);
    }
    // sum the cluster's partial tiles over this CTA's S rows, ranks in order, four features per 16-byte remote load
    uint32_t peer[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) peer[r] = r < csize ? sk_map_rank(part_addr, r) : 0u;
    const int S4 = S >> 2;                             // S is 16, 32, 64 or 128
    for (int idx = t; idx < S4 * NT; idx += 128) {
      const int m = idx / S4, f4 = idx - m * S4;
      const uint32_t off = uint32_t((m * kSkFeat + rank * S + f4 * 4) * 4);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < csize) {
          const float4 v = sk_ld_cluster4(peer[r] + off);
          a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
      }
      *reinterpret_cast<float4*>(red + m * S + f4 * 4) = a;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int outs = gated ? S / 2 : S;              // output features of this slice
    for (int idx = t; idx < outs * NT; idx += 128) {
      const int m = idx / outs, j = idx - m * outs;
      if (m >= p.M) continue;
      int n;
      float v;
      if (gated) {
        n = tile * 64 + rank * (S / 2) + j;
        float g = red[m * S + j], u = red[m * S + S / 2 + j];
        if (p.norm_eps >= 0.f) { g *= ss[m]; u *= ss[m]; }
        if (p.bias && n < p.N) { g += __bfloat162float(p.bias[n]); u += __bfloat162float(p.bias[p.up_offset + n]); }
        v = sk_gate(g, p.gate_kind) * u;
      } else {
        n = tile * kSkFeat + rank * S + j;
        v = red[m * S + j];
        if (p.norm_eps >= 0.f) v *= ss[m];
        if (p.bias && n < p.N) v += __bfloat162float(p.bias[n]);
      }
      if (n >= p.N) continue;
      if (p.residual) v += __bfloat162float(p.residual[size_t(m) * p.ldr + n]);
      p.C[size_t(m) * p.ldc + n] = __float2bfloat16(v);
    }
  }

  // nobody leaves while a peer may still read its shared memory
  __syncwarp();
  sk_cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, 64);
  }
}

template <int NT>
static int launch_skinny(const CUtensorMap& tmW, const CUtensorMap& tmX, const SkinnyParams& p, int tiles,
                         cudaStream_t stream) {
  using L = SkinnySmem<NT>;
  auto kern = skinny_gemm_kernel<NT>;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      }))
    return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(tiles * p.csize));
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(p.csize);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: this kernel's CTAs may start while the kernel before it in the stream drains; they
  // stop at pdl_wait() before their first read of global memory. IDRAK_PDL=0 launches the ordinary way.
  static const bool pdl = [] { const char* e = getenv("IDRAK_PDL"); return !(e && e[0] == '0'); }();
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  int rc = int(cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p));
  note_launches(1);
  return rc;
}

}  // namespace idrak

using namespace idrak;

// How many ways K is split (CTAs per cluster) for a product with `tiles` feature tiles and `kblocks` blocks of 64.
// IDRAK_SKINNY_SPLITS = 1 | 2 | 4 | 8 overrides the choice (for measurements), as far as K has that many blocks.
IDRAK_API int idrak_skinny_splits(int tiles, int kblocks) {
  const int slots = 2 * sm_count();
  if (const char* forced = getenv("IDRAK_SKINNY_SPLITS")) {
    const int f = atoi(forced);
    if (f == 1 || f == 2 || f == 4 || f == 8) {
      int c = f;
      while (c > 1 && kblocks < c) c >>= 1;
      return c;
    }
  }
  int c = 8;
  while (c > 1 && (tiles * c > slots || kblocks < c)) c >>= 1;     // measured: even one K block per CTA beats fewer CTAs
  return c;
}

// C[M, N] = epilogue(X[M, K] W^T), M <= 64. W is [N, K] (ldw elements per row), or with gate_kind >= 0 the stacked
// [gate; up] matrix of 2 * N rows and C = act(x Wg^T) * (x Wu^T). norm_eps >= 0 folds an RMS norm over K in (the norm
// weight must already be multiplied into W's columns). K % 8 == 0, rows 16-byte aligned. Returns 0, a CUDA error, or
// a negative argument error.
IDRAK_API int idrak_skinny_gemm(const void* X, int ldx, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                                const void* bias, const void* residual, int ldr, int gate_kind, float norm_eps,
                                void* stream_) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 64) return -2;
  if ((K & 7) || (ldx & 7) || (ldw & 7)) return -3;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return -4;
  if (gate_kind > 2) return -5;
  const bool gated = gate_kind >= 0;
  if (gated && (N % 8)) return -6;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  SkinnyParams p{};
  p.X = static_cast<const __nv_bfloat16*>(X); p.ldx = ldx;
  p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.M = M; p.N = N; p.K = K;
  p.gate_kind = gated ? gate_kind : -1;
  p.up_offset = gated ? N : 0;
  p.norm_eps = norm_eps;
  p.st = status_device_ptr();
  const int tiles = gated ? (N + 63) / 64 : (N + kSkFeat - 1) / kSkFeat;
  p.csize = idrak_skinny_splits(tiles, (K + kSkBK - 1) / kSkBK);
  const int NT = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const int w_rows = gated ? 2 * N : N;
  const int box_rows = gated ? (kSkFeat / p.csize) / 2 : kSkFeat;
  CUtensorMap tmW, tmX;
  {
    uint64_t dims[2] = {uint64_t(K), uint64_t(w_rows)};
    uint64_t strides[1] = {uint64_t(ldw) * 2};
    uint32_t box[2] = {uint32_t(kSkBK), uint32_t(box_rows)};
    if (encode_tensor_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(W), dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B))
      return -10;
  }
  {
    uint64_t dims[2] = {uint64_t(K), uint64_t(M)};
    uint64_t strides[1] = {uint64_t(ldx) * 2};
    uint32_t box[2] = {uint32_t(kSkBK), uint32_t(NT)};
    if (encode_tensor_map(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(X), dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B))
      return -11;
  }
  if (NT == 16) return launch_skinny<16>(tmW, tmX, p, tiles, stream);
  if (NT == 32) return launch_skinny<32>(tmW, tmX, p, tiles, stream);
  return launch_skinny<64>(tmW, tmX, p, tiles, stream);
}
