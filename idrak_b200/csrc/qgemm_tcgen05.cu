// GEMM over a frozen int8 / int4 weight, de-quantised on the way into shared memory (never materialised in bf16):
//   forward   y[M, N] = x[M, K] · W[K, N]           (W rows = inputs, columns = outputs)
//   backward  dx[M, K] = dy[M, N] · W[K, N]^T        (the same stored W read transposed)
// Weight formats (the reference's packed weights):
//   int8  one signed byte per value, row-major [K, N]; one scale per output column: w = q * scale[n]
//   int4  eight two's-complement nibbles (-8..7) per 32-bit word along a row (nibble c of word w is column 8w+c);
//         one scale per group of 32 input rows per column: w = q * scale[k / 32][n]
// Scales are fp16.
//
// Warp roles of the persistent CTA (448 threads):
//   warp 0        TMA producer of the activation tile (A, K-major, 128B swizzle)
//   warp 1        MMA issuer (tcgen05.mma, fp32 accumulators double-buffered in TMEM)
//   warps 2..5    epilogue (bias / GELU / residual / per-column int8 scale, TMA store) shared with the dense GEMM
//   warps 6..13   de-quantising producers of the weight tile: 128-bit (int8: 64-bit) coalesced loads of packed
//                 codes, convert to bf16 (int4: multiply by the group scale), store 16-byte chunks into the swizzled
//                 operand layout the tensor core reads (MN-major for forward, K-major for backward), then
//                 fence.proxy.async and arrive on the stage's barrier.
// For int8 forward the scale is constant along K and is applied once to the accumulator in the epilogue, so the
// codes enter the tensor core exactly; elsewhere the scale is applied in the producer.
//
// Reference counterparts: gemm_tc_nn_{int8w,int4w}_f32 (+_m64, _multi, _res, _gelu) and gemm_tc_nt_*w for the input
// gradient (src/Idrak.Gpu/Cuda/PtxKernels.TensorCore.cs:80-144), Int8Weight / Int4Weight
// (src/Idrak.Abstraction/Generation/Quantization.cs:382-470,659-1090).
#include "gemm_epilogue.cuh"
#include <cstring>

namespace idrak {

constexpr int kQThreads = 448;
constexpr int kQProducerWarps = 8;
constexpr int kQProducerThreads = kQProducerWarps * 32;

struct QWeight {
  const void* codes;       // int8: bytes [rows, ld]; int4: uint32 words [rows, ld_words]
  const __half* scales;    // int8: [cols]; int4: [ceil(rows / 32), scale_ld]
  int rows, cols;          // logical W is [rows = inputs, cols = outputs]
  int ld;                  // int8: bytes per row; int4: words per row
  int scale_ld;            // int4: scales per group row
  int bits;                // 8 or 4
  int scale_in_producer;   // int8: 1 when the scale cannot wait for the epilogue (transposed use)
};

template <int BN>
struct QSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kStagingBytes = 4 * 2 * 4096;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

// Eight consecutive codes of one weight row -> eight floats (scale applied when asked).
__device__ __forceinline__ void load_codes8(const QWeight& w, int row, int col, float (&out)[8]) {
  if (row >= w.rows || col >= w.cols) {
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = 0.f;
    return;
  }
  if (w.bits == 8) {
    const int8_t* p = static_cast<const int8_t*>(w.codes) + size_t(row) * w.ld + col;
    int8_t q[8];
    if (col + 8 <= w.cols && ((reinterpret_cast<uintptr_t>(p) & 7) == 0)) {
      *reinterpret_cast<uint2*>(q) = __ldg(reinterpret_cast<const uint2*>(p));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = (col + i < w.cols) ? p[i] : int8_t(0);
    }
    if (w.scale_in_producer) {
      const __half* sc = w.scales + col;
      if (col + 8 <= w.cols && (reinterpret_cast<uintptr_t>(sc) & 15) == 0) {
        const uint4 s4 = __ldg(reinterpret_cast<const uint4*>(sc));
        const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __half h = __ushort_as_half((unsigned short)((sw[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu));
          out[i] = float(q[i]) * __half2float(h);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = (col + i < w.cols) ? float(q[i]) * __half2float(w.scales[col + i]) : 0.f;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = float(q[i]);
    }
  } else {
    const uint32_t word = __ldg(static_cast<const uint32_t*>(w.codes) + size_t(row) * w.ld + (col >> 3));
    const __half* sc = w.scales + size_t(row >> 5) * w.scale_ld + col;
    if ((reinterpret_cast<uintptr_t>(sc) & 15) == 0) {
      // the scale rows are padded to eight columns: one 16-byte load brings the eight scales of this chunk
      const uint4 s4 = __ldg(reinterpret_cast<const uint4*>(sc));
      const uint32_t sw[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int q = int(word << (28 - 4 * i)) >> 28;        // sign-extended nibble i
        const __half h = __ushort_as_half((unsigned short)((sw[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu));
        out[i] = (col + i < w.cols) ? float(q) * __half2float(h) : 0.f;
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = int(word << (28 - 4 * i)) >> 28;          // sign-extended nibble i
      out[i] = (col + i < w.cols) ? float(q) * __half2float(sc[i]) : 0.f;
    }
  }
}

// kTrans = 0: forward  (B tile = W[k0 .. k0+64) x [n0 .. n0+BN), MN-major boxes of 64 columns)
// kTrans = 1: backward (B tile = W[o0 .. o0+BN) x [c0 .. c0+64), K-major: one 128-byte row per W row)
template <int BN, int kTrans>
__global__ void __launch_bounds__(kQThreads, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmC,
             const __grid_constant__ CUtensorMap tmAux, const GemmParams p, const QWeight w) {
  using L = QSmem<BN>;
  constexpr int kStages = L::kStages;
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
  const int k_blocks_total = (p.K + kBK - 1) / kBK;
  const int kb_per_split = (k_blocks_total + p.splits - 1) / p.splits;
  const int units = p.m_tiles * p.n_tiles * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1 + kQProducerWarps);    // the TMA arrive + one arrive per de-quantising warp
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
    // ------------------------------------------------------------------ activations by TMA
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      int stage = 0;
      uint32_t phase = 0;
      for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        int tm, tn, split;
        unit_to_tile(p, unit, tm, tn, split);
        const int kb0 = split * kb_per_split;
        const int kb1 = min(k_blocks_total, kb0 + kb_per_split);
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (5u << 16) | stage)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], L::kABytes);
          tma_load_2d(smem + stage * L::kStageBytes, &tmA, &full[stage], kb * kBK, tm * kBM);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
      if (*abort_flag) __nanosleep(50000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBM, BN, 0, kTrans ? 0 : 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++local) {
        int tm, tn, split;
        unit_to_tile(p, unit, tm, tn, split);
        const int kb0 = split * kb_per_split;
        const int kb1 = min(k_blocks_total, kb0 + kb_per_split);
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag, p.st, kTimeoutTmemEmpty, (5u << 16) | buf)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.st, kTimeoutSmemFull, (5u << 16) | stage)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            const uint64_t da = make_smem_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t db = kTrans ? make_smem_desc_sw128(sb + kk * 32, 16, 1024)
                                       : make_smem_desc_sw128(sb + kk * 2048, 8192, 1024);
            tc_mma_f16_ss(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&tmem_full[buf]);
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ de-quantising weight producers
    const int ptid = threadIdx.x - 6 * 32;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x) {
      int tm, tn, split;
      unit_to_tile(p, unit, tm, tn, split);
      const int kb0 = split * kb_per_split;
      const int kb1 = min(k_blocks_total, kb0 + kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (5u << 16) | (16 + stage))) {
          ok = false;
          break;
        }
        uint8_t* sb = smem + stage * L::kStageBytes + L::kABytes;
        if (kTrans == 0) {
          // tile rows = 64 inputs (k), BN/8 chunks of 8 outputs each
          constexpr int kChunks = BN / 8;
          const int row_base = kb * kBK, col_base = tn * BN;
#pragma unroll 2
          for (int i = ptid; i < 64 * kChunks; i += kQProducerThreads) {
            const int r = i / kChunks, c8 = i - r * kChunks;
            float v[8];
            load_codes8(w, row_base + r, col_base + c8 * 8, v);
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(sb + (c8 >> 3) * 8192 + r * 128 + (((c8 & 7) ^ (r & 7)) << 4)) = o;
          }
        } else {
          // tile rows = BN outputs of this product (rows of W), 8 chunks of 8 contraction values (columns of W)
          const int row_base = tn * BN, col_base = kb * kBK;
#pragma unroll 2
          for (int i = ptid; i < BN * 8; i += kQProducerThreads) {
            const int r = i >> 3, c8 = i & 7;
            float v[8];
            load_codes8(w, row_base + r, col_base + c8 * 8, v);
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(sb + r * 128 + ((c8 ^ (r & 7)) << 4)) = o;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[stage]);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps, 128 rows)
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    int local = 0;
    int ring = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++local) {
      int tm, tn, split;
      unit_to_tile(p, unit, tm, tn, split);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[buf], acc_phase, abort_flag, p.st, kTimeoutTmemFull, (5u << 16) | buf)) break;
      tc_fence_after();
      const int row = tm * kBM + row_in_tile;
      const int n0 = tn * BN;
      if (p.tma_store && p.splits == 1) {
        const int row0 = tm * kBM + quarter * 32;
        const bool gelu = (p.act == kActGelu);
        uint8_t* my_stage = staging + quarter * 2 * 4096;
#pragma unroll 1
        for (int s64 = 0; s64 < BN / 64; ++s64) {
          const int col0 = n0 + s64 * 64;
          if (col0 >= p.N || row0 >= p.M) break;
          uint8_t* cbuf = my_stage + (gelu ? 0 : (ring & 1)) * 4096;
          uint8_t* abuf = my_stage + 4096;
          if (lane == 0) {
            if (gelu) tma_store_wait_read<0>(); else tma_store_wait_read<1>();
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
              if (row < p.M && col < p.N) epilogue_math8(p, row, col, v, min(8, p.N - col), false, pre);
              const int chunk = ((h * 4 + g) ^ (lane & 7)) << 4;
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(cbuf + lane * 128 + chunk) = o;
              if (gelu) {
                uint4 a;
                a.x = pack_bf16x2(pre[0], pre[1]); a.y = pack_bf16x2(pre[2], pre[3]);
                a.z = pack_bf16x2(pre[4], pre[5]); a.w = pack_bf16x2(pre[6], pre[7]);
                *reinterpret_cast<uint4*>(abuf + lane * 128 + chunk) = a;
              }
            }
          }
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
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN + c * 32, r);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row < p.M && col0 < p.N) {
            if (p.splits > 1) {
              float* ws = p.workspace + (size_t(split) * p.M + row) * p.N + col0;
              for (int i = 0; i < 32 && col0 + i < p.N; ++i) ws[i] = __uint_as_float(r[i]);
            } else {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int col = col0 + g * 8;
                if (col < p.N) {
                  float v[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]) * p.alpha;
                  epilogue8(p, row, col, v, min(8, p.N - col));
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[buf]);
    }
    if (p.tma_store && lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// partial sums of split-K -> epilogue (same contract as the dense GEMM's reducer)
__global__ void __launch_bounds__(256) qsplitk_reduce_kernel(const GemmParams p) {
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
      const float* ws = p.workspace + (size_t(s) * p.M + row) * p.N + col;
      for (int j = 0; j < nvalid; ++j) v[j] += ws[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= p.alpha;
    epilogue8(p, row, col, v, nvalid);
  }
}

template <int BN, int kTrans>
static int launch_q(const CUtensorMap& tmA, const CUtensorMap& tmC, const CUtensorMap& tmAux, const GemmParams& p,
                    const QWeight& w, int grid, cudaStream_t stream) {
  using L = QSmem<BN>;
  auto kern = qgemm_kernel<BN, kTrans>;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      }))
    return e;
  kern<<<grid, kQThreads, L::kTotal, stream>>>(tmA, tmC, tmAux, p, w);
  note_launches(1);
  return int(cudaGetLastError());
}

// plain de-quantisation to bf16 (checks, merges, exports)
__global__ void qdequant_kernel(QWeight w, __nv_bfloat16* __restrict__ out, int ld_out) {
  const int chunks = (w.cols + 7) / 8;
  const long long total = (long long)w.rows * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / chunks), c = int(i - (long long)r * chunks) * 8;
    float v[8];
    load_codes8(w, r, c, v);
    __nv_bfloat16* o = out + size_t(r) * ld_out + c;
    if (c + 8 <= w.cols && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
      uint4 q;                                            // one 16-byte store per eight columns
      q.x = pack_bf16x2(v[0], v[1]); q.y = pack_bf16x2(v[2], v[3]);
      q.z = pack_bf16x2(v[4], v[5]); q.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(o) = q;
    } else {
      for (int j = 0; j < 8 && c + j < w.cols; ++j) o[j] = __float2bfloat16(v[j]);
    }
  }
}

}  // namespace idrak

using namespace idrak;

// y = epilogue(alpha * x · W)            (transposed = 0; x is [M, rows], y is [M, cols])
// y = epilogue(alpha * x · W^T)          (transposed = 1; x is [M, cols], y is [M, rows])
// codes / scales describe W as stored ([rows = inputs, cols = outputs], see the file header); bits = 8 or 4.
IDRAK_API int idrak_qgemm(const void* x, int ldx, const void* codes, const void* scales, int w_rows, int w_cols,
                          int w_ld, int scale_ld, int bits, int transposed, void* C, int ldc, int c_fp32, int M,
                          const void* bias, const void* residual, int ldr, int act, void* aux, int ld_aux, int beta,
                          float alpha, int splits, float* workspace, void* stream_) {
  if (bits != 8 && bits != 4) return -2;
  if (ldx & 7) return -3;
  if (act != kActNone && aux == nullptr) return -4;
  const int N = transposed ? w_rows : w_cols;
  const int K = transposed ? w_cols : w_rows;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int bn = (N <= 128) ? 128 : 256;
  GemmParams p{};
  memset(&p, 0, sizeof(p));
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
    const int kblocks = (K + kBK - 1) / kBK;
    if (p.splits > kblocks) p.splits = kblocks;
    const int per = (kblocks + p.splits - 1) / p.splits;
    p.splits = (kblocks + per - 1) / per;
  }
  p.workspace = workspace;
  p.m_tiles = (M + kBM - 1) / kBM;
  p.n_tiles = (N + bn - 1) / bn;
  p.st = status_device_ptr();
  QWeight w;
  w.codes = codes;
  w.scales = static_cast<const __half*>(scales);
  w.rows = w_rows; w.cols = w_cols; w.ld = w_ld; w.scale_ld = scale_ld; w.bits = bits;
  w.scale_in_producer = (bits == 8 && transposed) ? 1 : 0;
  p.col_scale = (bits == 8 && !transposed) ? w.scales : nullptr;

  CUtensorMap tmA, tmC, tmAux;
  memset(&tmC, 0, sizeof(tmC));
  memset(&tmAux, 0, sizeof(tmAux));
  {
    uint64_t dims[2] = {uint64_t(K), uint64_t(M)};
    uint64_t str[1] = {uint64_t(ldx) * 2};
    uint32_t box[2] = {kBK, kBM};
    if (encode_tensor_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, str, box,
                          CU_TENSOR_MAP_SWIZZLE_128B))
      return -10;
  }
  p.tma_store = 0;
  if (!c_fp32 && !beta && p.splits == 1 && (ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
      (act != kActGelu || ((ld_aux % 8) == 0 && (reinterpret_cast<uintptr_t>(aux) & 15) == 0))) {
    uint64_t dims[2] = {uint64_t(N), uint64_t(M)};
    uint32_t box[2] = {64, 32};
    uint64_t str_c[1] = {uint64_t(ldc) * 2};
    int ok = encode_tensor_map(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dims, str_c, box,
                               CU_TENSOR_MAP_SWIZZLE_128B) == 0;
    if (ok && act == kActGelu) {
      uint64_t str_a[1] = {uint64_t(ld_aux) * 2};
      ok = encode_tensor_map(&tmAux, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, aux, dims, str_a, box,
                             CU_TENSOR_MAP_SWIZZLE_128B) == 0;
    }
    p.tma_store = ok ? 1 : 0;
  }
  const int units = p.m_tiles * p.n_tiles * p.splits;
  const int grid = units < sm_count() ? units : sm_count();
  int rc;
  if (bn == 256) rc = transposed ? launch_q<256, 1>(tmA, tmC, tmAux, p, w, grid, stream)
                                 : launch_q<256, 0>(tmA, tmC, tmAux, p, w, grid, stream);
  else rc = transposed ? launch_q<128, 1>(tmA, tmC, tmAux, p, w, grid, stream)
                       : launch_q<128, 0>(tmA, tmC, tmAux, p, w, grid, stream);
  if (rc) return rc;
  if (p.splits > 1) {
    const long long groups = (long long)M * ((N + 7) / 8);
    long long want = (groups + 255) / 256, cap = (long long)sm_count() * 8;
    qsplitk_reduce_kernel<<<int(want < cap ? want : cap), 256, 0, stream>>>(p);
    note_launches(1);
    rc = int(cudaGetLastError());
  }
  return rc;
}

IDRAK_API int idrak_qdequant(const void* codes, const void* scales, int w_rows, int w_cols, int w_ld, int scale_ld,
                             int bits, void* out, int ld_out, void* stream_) {
  QWeight w;
  w.codes = codes;
  w.scales = static_cast<const __half*>(scales);
  w.rows = w_rows; w.cols = w_cols; w.ld = w_ld; w.scale_ld = scale_ld; w.bits = bits;
  w.scale_in_producer = 1;
  const long long total = (long long)w_rows * ((w_cols + 7) / 8);
  long long want = (total + 255) / 256, cap = (long long)sm_count() * 16;
  qdequant_kernel<<<int(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      w, static_cast<__nv_bfloat16*>(out), ld_out);
  note_launches(1);
  return int(cudaGetLastError());
}
