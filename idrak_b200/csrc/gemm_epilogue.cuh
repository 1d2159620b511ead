// Pieces shared by the dense and the dequant-fused GEMM kernels: tile constants, the parameter block, the fused
// epilogue (bias, GELU / GELU', residual, accumulate, bf16 or fp32 store) and the tile rasterisation.
#pragma once
#include "common.cuh"

namespace idrak {

constexpr int kBM = 128;
constexpr int kBK = 64;          // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;
constexpr int kGroupM = 16;      // raster: 16 row-tiles share the resident column tiles in L2

enum GemmAct : int { kActNone = 0, kActGelu = 1, kActGeluGrad = 2 };

struct GemmParams {
  int M, N, K;
  void* C;              // bf16 or fp32 [M, ldc]
  int ldc;
  int c_fp32;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  int ldr;
  int act;                        // GemmAct
  __nv_bfloat16* aux;             // kActGelu: pre-activation out; kActGeluGrad: pre-activation in. [M, ld_aux]
  int ld_aux;
  int beta;                       // 1: add the old contents of C
  float alpha;                    // scale on the accumulator
  int splits;                     // split-K factor (1 = direct epilogue)
  float* workspace;               // [splits, M, N] fp32 when splits > 1
  int m_tiles, n_tiles;
  int tma_store;                  // 1: bf16 C (and aux) leave through shared-memory staging + TMA stores
  const __half* col_scale;        // [N] per-column factor applied to the accumulator first (int8 weights), or null
  Status* st;
};

// Element-wise part of the epilogue on 8 consecutive columns of one row: bias, activation, residual.
// `v` holds alpha-scaled accumulators on entry and the values to store on return. With kActGelu the
// pre-activation goes to `pre` (rounded to bf16 like the stored copy) and, when `store_aux`, to p.aux.
__device__ __forceinline__ void epilogue_math8(const GemmParams& p, int row, int col, float (&v)[8], int nvalid,
                                               bool store_aux, float (&pre)[8]) {
  const bool vec = (nvalid == 8);
  if (p.col_scale) {
    for (int i = 0; i < nvalid; ++i) v[i] *= __half2float(p.col_scale[col + i]);
  }
  if (p.bias) {
    if (vec && ((reinterpret_cast<uintptr_t>(p.bias + col) & 15) == 0)) {
      uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
      float2 f;
      f = unpack_bf16x2(b.x); v[0] += f.x; v[1] += f.y;
      f = unpack_bf16x2(b.y); v[2] += f.x; v[3] += f.y;
      f = unpack_bf16x2(b.z); v[4] += f.x; v[5] += f.y;
      f = unpack_bf16x2(b.w); v[6] += f.x; v[7] += f.y;
    } else {
      for (int i = 0; i < nvalid; ++i) v[i] += __bfloat162float(p.bias[col + i]);
    }
  }
  if (p.act != kActNone) {
    __nv_bfloat16* ax = p.aux + size_t(row) * p.ld_aux + col;
    const bool axvec = vec && ((reinterpret_cast<uintptr_t>(ax) & 15) == 0);
    if (p.act == kActGelu) {
      if (store_aux) {
        if (axvec) {
          uint4 o;
          o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
          o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
          *reinterpret_cast<uint4*>(ax) = o;
        } else {
          for (int i = 0; i < nvalid; ++i) ax[i] = __float2bfloat16(v[i]);
        }
      }
      // the activation sees the value as it was stored (bf16), so forward and backward agree
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        pre[i] = __bfloat162float(__float2bfloat16(v[i]));
        v[i] = gelu_tanh(pre[i]);
      }
    } else {
      float x[8];
      if (axvec) {
        uint4 a = *reinterpret_cast<const uint4*>(ax);
        float2 f;
        f = unpack_bf16x2(a.x); x[0] = f.x; x[1] = f.y;
        f = unpack_bf16x2(a.y); x[2] = f.x; x[3] = f.y;
        f = unpack_bf16x2(a.z); x[4] = f.x; x[5] = f.y;
        f = unpack_bf16x2(a.w); x[6] = f.x; x[7] = f.y;
      } else {
        for (int i = 0; i < 8; ++i) x[i] = i < nvalid ? __bfloat162float(ax[i]) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= gelu_tanh_grad(x[i]);
    }
  }
  if (p.residual) {
    const __nv_bfloat16* r = p.residual + size_t(row) * p.ldr + col;
    if (vec && ((reinterpret_cast<uintptr_t>(r) & 15) == 0)) {
      uint4 a = *reinterpret_cast<const uint4*>(r);
      float2 f;
      f = unpack_bf16x2(a.x); v[0] += f.x; v[1] += f.y;
      f = unpack_bf16x2(a.y); v[2] += f.x; v[3] += f.y;
      f = unpack_bf16x2(a.z); v[4] += f.x; v[5] += f.y;
      f = unpack_bf16x2(a.w); v[6] += f.x; v[7] += f.y;
    } else {
      for (int i = 0; i < nvalid; ++i) v[i] += __bfloat162float(r[i]);
    }
  }
}

// Full epilogue with direct global stores (any alignment, fp32 or bf16 output, optional accumulate).
__device__ __forceinline__ void epilogue8(const GemmParams& p, int row, int col, float (&v)[8], int nvalid) {
  const bool vec = (nvalid == 8);
  float pre[8];
  epilogue_math8(p, row, col, v, nvalid, true, pre);
  if (p.c_fp32) {
    float* c = reinterpret_cast<float*>(p.C) + size_t(row) * p.ldc + col;
    if (vec && ((reinterpret_cast<uintptr_t>(c) & 15) == 0)) {
      float4* c4 = reinterpret_cast<float4*>(c);
      if (p.beta) {
        float4 o0 = c4[0], o1 = c4[1];
        v[0] += o0.x; v[1] += o0.y; v[2] += o0.z; v[3] += o0.w;
        v[4] += o1.x; v[5] += o1.y; v[6] += o1.z; v[7] += o1.w;
      }
      c4[0] = make_float4(v[0], v[1], v[2], v[3]);
      c4[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      for (int i = 0; i < nvalid; ++i) c[i] = p.beta ? c[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc + col;
    if (vec && ((reinterpret_cast<uintptr_t>(c) & 15) == 0)) {
      if (p.beta) {
        uint4 a = *reinterpret_cast<const uint4*>(c);
        float2 f;
        f = unpack_bf16x2(a.x); v[0] += f.x; v[1] += f.y;
        f = unpack_bf16x2(a.y); v[2] += f.x; v[3] += f.y;
        f = unpack_bf16x2(a.z); v[4] += f.x; v[5] += f.y;
        f = unpack_bf16x2(a.w); v[6] += f.x; v[7] += f.y;
      }
      uint4 o;
      o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
      o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(c) = o;
    } else {
      for (int i = 0; i < nvalid; ++i) {
        float o = v[i] + (p.beta ? __bfloat162float(c[i]) : 0.f);
        c[i] = __float2bfloat16(o);
      }
    }
  }
}

__device__ __forceinline__ void unit_to_tile(const GemmParams& p, int unit, int& tm, int& tn, int& split) {
  const int tiles = p.m_tiles * p.n_tiles;
  split = unit / tiles;
  int t = unit - split * tiles;
  const int per_group = kGroupM * p.n_tiles;
  int group = t / per_group;
  int first_m = group * kGroupM;
  int gsz = min(p.m_tiles - first_m, kGroupM);
  int r = t - group * per_group;
  tm = first_m + (r % gsz);
  tn = r / gsz;
}
// The CTA-pair kernel (gemm2_tcgen05.cu): whether a product should use it, and its launcher.
bool gemm_pair_wanted(int M, int N, int K, int splits);
int gemm_pair_launch(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, const CUtensorMap& tmC,
                     const CUtensorMap& tmAux, GemmParams p, int fp16, cudaStream_t stream);
}  // namespace idrak
