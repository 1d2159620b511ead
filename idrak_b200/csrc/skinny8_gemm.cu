// Few-row products over int8 weights (one scale per output feature): C[M, N] = X[M, K] (W8[N, K] * scale[N])^T with
// M <= 64 tokens, bound by streaming the weight codes once - half the bytes of the bf16 product.
//
// Same shape of kernel as the bf16 few-row product (skinny_gemm.cu): the weights fill the 128-row side of a tcgen05
// tile, the tokens the narrow side, K is split over a cluster of up to 8 CTAs whose partial tiles are summed through
// distributed shared memory in rank order. What differs is the operand path. The codes are stored K-major ([N, K] int8,
// the transposed copy a packed weight makes for decoding) and arrive by TMA as a [128, 64]-byte tile in a staging
// buffer; the four warps that later run the epilogue turn each tile into the bf16 operand tile the tensor core reads
// (128-byte swizzled rows of 64 bf16) while the next tiles are in flight, and hand it to the MMA thread through a
// barrier of their own. The scale of a feature multiplies its accumulator row in the epilogue, so the conversion is a
// plain int8 -> bf16 (exact). Per stage: bf16 operand tile 16 KB, token rows 8 KB, codes 8 KB = 32 KB, three stages,
// two CTAs per SM.
//
//   warp 0      TMA producer (codes and token rows of this CTA's K range)
//   warp 1      MMA issuer (waits for "converted", not for the TMA barrier)
//   warps 2..5  convert codes -> bf16 per K block, then move the accumulator to shared memory, meet the cluster, reduce
//               their slice and run the epilogue: scale, bias, residual, or act(gate) * up for a stacked gate / up matrix
//
// Every mbarrier wait is bounded (status word + abort flag) and every thread reaches both cluster barriers.
//
// Reference counterparts: int8_gemv_f32 and its fused forms (src/Idrak.Gpu/Cuda/PtxKernels.Quantized.cs:13,454-495).
#include "common.cuh"
#include <cstdlib>

namespace idrak {

constexpr int kS8Feat = 128;
constexpr int kS8BK = 64;
constexpr int kS8Stages = 3;
constexpr int kS8Threads = 192;

struct Skinny8Params {
  const __nv_bfloat16* X;
  int ldx;
  const __half* scales;          // [rows of W8]: one per output feature (gated: gate rows then up rows)
  __nv_bfloat16* C;
  int ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int ldr;
  int M, N, K;
  int gate_kind;                 // -1 plain; 0 silu, 1 gelu (tanh), 2 relu
  int up_offset;
  int csize;
  Status* st;
};

struct Skinny8Smem {
  static constexpr int kWb = kS8Feat * kS8BK * 2;           // 16 KB bf16 operand tile
  static constexpr int kXs = 64 * kS8BK * 2;                // 8 KB token rows (sized for 64 tokens)
  static constexpr int kW8 = kS8Feat * kS8BK;               // 8 KB codes
  static constexpr int kStage = kWb + kXs + kW8;            // 32 KB
  static constexpr int kPart = 0;                           // after the main loop: partial tile [NT][128] fp32
  static constexpr int kRed = 32768;                        // and this CTA's reduced slice
  static constexpr int kBar = kS8Stages * kStage;
  static constexpr int kTotal = kBar + 256 + 1024;
};

__device__ __forceinline__ uint32_t s8_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t s8_map_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ float s8_ld_cluster(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 s8_ld_cluster4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void s8_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float s8_gate(float g, int kind) {
  if (kind == 0) return g / (1.f + __expf(-g));
  if (kind == 1) return gelu_tanh(g);
  return fmaxf(g, 0.f);
}
// four int8 codes (one 32-bit word) -> two packed bf16 pairs, without the integer-to-float unit (a quarter-rate pipe
// that would bound the kernel): code + 128 is dropped into the mantissa of 2^23 by one byte permute, and subtracting
// 2^23 + 128 on the FP32 pipe leaves the code's value exactly.
__device__ __forceinline__ void s8_cvt4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t x = w ^ 0x80808080u;
  const float bias = 8388736.f;                        // 2^23 + 128
  const float f0 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650)) - bias;
  const float f1 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7651)) - bias;
  const float f2 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7652)) - bias;
  const float f3 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7653)) - bias;
  lo = pack_bf16x2(f0, f1);
  hi = pack_bf16x2(f2, f3);
}

template <int NT>
__global__ void __launch_bounds__(kS8Threads, 2)
skinny8_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    const Skinny8Params p) {
  using L = Skinny8Smem;
  constexpr int kXbytes = NT * kS8BK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* part = reinterpret_cast<float*>(smem + L::kPart);
  float* red = reinterpret_cast<float*>(smem + L::kRed);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* conv = full + kS8Stages;
  uint64_t* empty = conv + kS8Stages;
  uint64_t* acc_full = empty + kS8Stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int csize = p.csize;
  const int rank = int(s8_cluster_rank());
  const int tile = blockIdx.x / csize;
  const int S = kS8Feat / csize;
  const bool gated = p.gate_kind >= 0;
  const int kblocks = (p.K + kS8BK - 1) / kS8BK;
  const int per = (kblocks + csize - 1) / csize;
  const int kb0 = min(kblocks, rank * per), kb1 = min(kblocks, kb0 + per);

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kS8Stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&conv[s], 128);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_acc = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, issued_phase = 0;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (9u << 16) | stage)) {
          ok = false;
          break;
        }
        uint8_t* base = smem + stage * L::kStage;
        uint8_t* sx = base + L::kWb;
        uint8_t* s8 = sx + L::kXs;
        mbar_expect_tx(&full[stage], L::kW8 + kXbytes);
        if (!gated) {
          tma_load_2d(s8, &tmW, &full[stage], kb * kS8BK, tile * kS8Feat);
        } else {
          const int half = S / 2;
          for (int r = 0; r < csize; ++r) {
            const int f = tile * 64 + r * half;
            tma_load_2d(s8 + (r * S) * kS8BK, &tmW, &full[stage], kb * kS8BK, f);
            tma_load_2d(s8 + (r * S + half) * kS8BK, &tmW, &full[stage], kb * kS8BK, p.up_offset + f);
          }
        }
        tma_load_2d(sx, &tmX, &full[stage], kb * kS8BK, 0);
        issued_mask |= 1u << stage;
        issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
        if (++stage == kS8Stages) { stage = 0; phase ^= 1; }
      }
      if (!ok || *abort_flag) {
        for (int s = 0; s < kS8Stages; ++s) {
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
      constexpr uint32_t idesc = make_idesc_f16(kS8Feat, NT, 0, 0, 1);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (!mbar_wait(&conv[stage], phase, abort_flag, p.st, kTimeoutSmemFull, (9u << 16) | (8 + stage))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sw = smem_u32(smem + stage * L::kStage);
        const uint32_t sx = sw + L::kWb;
#pragma unroll
        for (int kk = 0; kk < kS8BK / 16; ++kk) {
          const uint64_t da = make_smem_desc_sw128(sw + kk * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sx + kk * 32, 16, 1024);
          tc_mma_f16_ss(tmem_acc, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&empty[stage]);
        if (++stage == kS8Stages) { stage = 0; phase ^= 1; }
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    // ---------------------------------------------------------------- converter warps: codes -> bf16 operand tiles
    const int t = threadIdx.x - 64;                   // 0 .. 127 = row of the tile
    {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (ok && !mbar_wait(&full[stage], phase, abort_flag, p.st, kTimeoutSmemFull, (9u << 16) | (16 + stage))) ok = false;
        uint8_t* base = smem + stage * L::kStage;
        if (ok) {
          // the staged tile is 512 chunks of 16 codes; neighbouring threads take neighbouring chunks (no bank conflicts
          // on the read), each chunk becomes two 16-byte chunks of 8 bf16 in the swizzled operand row
          const uint4* src = reinterpret_cast<const uint4*>(base + L::kWb + L::kXs);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int i = c * 128 + t;
            const int r = i >> 2, ch = i & 3;
            const uint4 q = src[i];
            uint4 a, b;
            s8_cvt4(q.x, a.x, a.y);
            s8_cvt4(q.y, a.z, a.w);
            s8_cvt4(q.z, b.x, b.y);
            s8_cvt4(q.w, b.z, b.w);
            uint8_t* dst = base + r * 128;
            *reinterpret_cast<uint4*>(dst + (((2 * ch) ^ (r & 7)) << 4)) = a;
            *reinterpret_cast<uint4*>(dst + (((2 * ch + 1) ^ (r & 7)) << 4)) = b;
          }
          fence_proxy_async_smem();                    // the tensor core reads these through the async proxy
        }
        mbar_arrive(&conv[stage]);                     // arrive even after a failure so the MMA thread is not left waiting
        if (++stage == kS8Stages) { stage = 0; phase ^= 1; }
      }
    }
    const bool have = kb1 > kb0;
    if (have && ok) ok = mbar_wait(acc_full, 0, abort_flag, p.st, kTimeoutTmemFull, (9u << 16) | 32);
    tc_fence_after();
    const int q = warp & 3;
    const int f = q * 32 + lane;
    if (have && ok) {
#pragma unroll
      for (int c = 0; c < NT / 16; ++c) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(tmem_acc + (uint32_t(q * 32) << 16) + c * 16, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) part[(c * 16 + i) * kS8Feat + f] = __uint_as_float(v[i]);
      }
    } else {
      for (int m = 0; m < NT; ++m) part[m * kS8Feat + f] = 0.f;
    }
  }

  tc_fence_before();
  __syncwarp();
  s8_cluster_sync();

  if (warp >= 2) {
    const int t = threadIdx.x - 64;
    const uint32_t part_addr = smem_u32(part);
    // sum the cluster's partial tiles over this CTA's S rows, ranks in order, four features per 16-byte remote load
    uint32_t peer[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) peer[r] = r < csize ? s8_map_rank(part_addr, r) : 0u;
    const int S4 = S >> 2;                             // S is 16, 32, 64 or 128
    for (int idx = t; idx < S4 * NT; idx += 128) {
      const int m = idx / S4, f4 = idx - m * S4;
      const uint32_t off = uint32_t((m * kS8Feat + rank * S + f4 * 4) * 4);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < csize) {
          const float4 v = s8_ld_cluster4(peer[r] + off);
          a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
      }
      *reinterpret_cast<float4*>(red + m * S + f4 * 4) = a;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int outs = gated ? S / 2 : S;
    for (int idx = t; idx < outs * NT; idx += 128) {
      const int m = idx / outs, j = idx - m * outs;
      if (m >= p.M) continue;
      int n;
      float v;
      if (gated) {
        n = tile * 64 + rank * (S / 2) + j;
        if (n >= p.N) continue;
        float g = red[m * S + j] * __half2float(p.scales[n]);
        float u = red[m * S + S / 2 + j] * __half2float(p.scales[p.up_offset + n]);
        if (p.bias) { g += __bfloat162float(p.bias[n]); u += __bfloat162float(p.bias[p.up_offset + n]); }
        v = s8_gate(g, p.gate_kind) * u;
      } else {
        n = tile * kS8Feat + rank * S + j;
        if (n >= p.N) continue;
        v = red[m * S + j] * __half2float(p.scales[n]);
        if (p.bias) v += __bfloat162float(p.bias[n]);
      }
      if (p.residual) v += __bfloat162float(p.residual[size_t(m) * p.ldr + n]);
      p.C[size_t(m) * p.ldc + n] = __float2bfloat16(v);
    }
  }

  __syncwarp();
  s8_cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, 64);
  }
}

template <int NT>
static int launch_skinny8(const CUtensorMap& tmW, const CUtensorMap& tmX, const Skinny8Params& p, int tiles,
                          cudaStream_t stream) {
  using L = Skinny8Smem;
  auto kern = skinny8_gemm_kernel<NT>;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      }))
    return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(tiles * p.csize));
  cfg.blockDim = dim3(kS8Threads);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(p.csize);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int rc = int(cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p));
  note_launches(1);
  return rc;
}

}  // namespace idrak

using namespace idrak;

extern "C" int idrak_skinny_splits(int tiles, int kblocks);

// C[M, N] = epilogue(X[M, K] (W8 * scale)^T), M <= 64. W8 is [N, K] int8 codes, K-major, ldw bytes per row (a multiple
// of 16); scales one fp16 per row of W8. With gate_kind >= 0, W8 is the stacked [gate; up] matrix of 2 * N rows and
// C = act(gate) * up. K % 16 == 0. Returns 0, a CUDA error, or a negative argument error.
IDRAK_API int idrak_skinny8_gemm(const void* X, int ldx, const void* W8, int ldw, const void* scales, void* C, int ldc,
                                 int M, int N, int K, const void* bias, const void* residual, int ldr, int gate_kind,
                                 void* stream_) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 64) return -2;
  if ((K & 15) || (ldx & 7) || (ldw & 15)) return -3;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W8) & 15)) return -4;
  if (gate_kind > 2) return -5;
  const bool gated = gate_kind >= 0;
  if (gated && (N % 8)) return -6;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  Skinny8Params p{};
  p.X = static_cast<const __nv_bfloat16*>(X); p.ldx = ldx;
  p.scales = static_cast<const __half*>(scales);
  p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.M = M; p.N = N; p.K = K;
  p.gate_kind = gated ? gate_kind : -1;
  p.up_offset = gated ? N : 0;
  p.st = status_device_ptr();
  const int tiles = gated ? (N + 63) / 64 : (N + kS8Feat - 1) / kS8Feat;
  p.csize = idrak_skinny_splits(tiles, (K + kS8BK - 1) / kS8BK);
  const int NT = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const int w_rows = gated ? 2 * N : N;
  const int box_rows = gated ? (kS8Feat / p.csize) / 2 : kS8Feat;
  CUtensorMap tmW, tmX;
  {
    uint64_t dims[2] = {uint64_t(K), uint64_t(w_rows)};
    uint64_t strides[1] = {uint64_t(ldw)};
    uint32_t box[2] = {uint32_t(kS8BK), uint32_t(box_rows)};
    if (encode_tensor_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(W8), dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_NONE))
      return -10;
  }
  {
    uint64_t dims[2] = {uint64_t(K), uint64_t(M)};
    uint64_t strides[1] = {uint64_t(ldx) * 2};
    uint32_t box[2] = {uint32_t(kS8BK), uint32_t(NT)};
    if (encode_tensor_map(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(X), dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B))
      return -11;
  }
  if (NT == 16) return launch_skinny8<16>(tmW, tmX, p, tiles, stream);
  if (NT == 32) return launch_skinny8<32>(tmW, tmX, p, tiles, stream);
  return launch_skinny8<64>(tmW, tmX, p, tiles, stream);
}
