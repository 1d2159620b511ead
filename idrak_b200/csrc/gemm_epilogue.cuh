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

// kActGelu / kActGeluGrad: C = gelu(v) with the pre-activation saved in aux / C = v * gelu'(aux).
// kActGeluD / kActMulAux: the same layer with the derivative taken in the forward pass, where the tanh is at hand
// anyway: C = gelu(v) and aux = gelu'(v) / C = v * aux. The backward epilogue is then one multiply.
enum GemmAct : int { kActNone = 0, kActGelu = 1, kActGeluGrad = 2, kActGeluD = 3, kActMulAux = 4 };

struct GemmParams {
  int M, N, K;
  void* C;              // bf16 or fp32 [M, ldc]
  int ldc;
  int c_fp32;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  int ldr;
  int act;                        // GemmAct
  __nv_bfloat16* aux;             // kActGelu: pre-activation out; kActGeluGrad: pre-activation in; kActGeluD:
                                  // derivative out; kActMulAux: factor in. [M, ld_aux]
  int ld_aux;
  int beta;                       // 1: add the old contents of C
  float alpha;                    // scale on the accumulator
  int splits;                     // split-K factor (1 = direct epilogue)
  float* workspace;               // [splits, M, N] fp32 when splits > 1
  int m_tiles, n_tiles;
  int tma_store;                  // 1: bf16 C (and aux) leave through shared-memory staging + TMA stores
  const __half* col_scale;        // [N] per-column factor applied to the accumulator first (int8 weights), or null
  const float* row_scale_f;       // [M] and
  const float* col_scale_f;       // [N] fp32 factors on the accumulator (8-bit operands quantised per row), or null
  unsigned long long* prof;       // role timers [grid][8] (cycles), or null: see idrak_gemm_role_timers
  int epi_mode;                   // EpiMode: which compile-time variant of the staged epilogue fits this product
  Status* st;
  // grouped products (mixture of experts): rows sorted by expert in segments padded to 128 rows
  const int* tile_group;          // per-row-tile mode: expert of every 128-row M tile
  const int* tiles_in_use;        // per-row-tile mode: device scalar, M tiles that hold rows (the rest are skipped)
  int group_b_rows;               // per-row-tile mode: rows of one expert in the stacked B array
  const int* group_kb;            // per-expert-K mode: [groups + 1] bounds of each expert's rows in 64-row blocks
  int groups;                     // per-expert-K mode: experts; C is the stacked [groups * M_per, N] array
  int extra_kb;                   // second operand pair (low-rank term): its K extent in 64-element blocks, else 0
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
  if (p.row_scale_f) {
    const float rs = p.row_scale_f[row];
    for (int i = 0; i < nvalid; ++i) v[i] *= rs * p.col_scale_f[col + i];
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
    if (p.act == kActGelu || p.act == kActGeluD) {
      if (p.act == kActGeluD) {
        // value and derivative from the unrounded pre-activation; `pre` carries the derivative
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float g, d;
          gelu_tanh_both(v[i], g, d);
          v[i] = g;
          pre[i] = d;
        }
      } else {
        // the activation sees the value as it is stored (bf16), so forward and backward agree
#pragma unroll
        for (int i = 0; i < 8; ++i) pre[i] = __bfloat162float(__float2bfloat16(v[i]));
      }
      if (store_aux) {
        if (axvec) {
          uint4 o;
          o.x = pack_bf16x2(pre[0], pre[1]); o.y = pack_bf16x2(pre[2], pre[3]);
          o.z = pack_bf16x2(pre[4], pre[5]); o.w = pack_bf16x2(pre[6], pre[7]);
          *reinterpret_cast<uint4*>(ax) = o;
        } else {
          for (int i = 0; i < nvalid; ++i) ax[i] = __float2bfloat16(pre[i]);
        }
      }
      if (p.act == kActGelu) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = gelu_tanh(pre[i]);
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
      if (p.act == kActMulAux) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= x[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] *= gelu_tanh_grad(x[i]);
      }
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

__device__ __forceinline__ void unit_to_tile_n(int m_tiles, int n_tiles, int unit, int& tm, int& tn, int& split) {
  const int tiles = m_tiles * n_tiles;
  split = unit / tiles;
  int t = unit - split * tiles;
  const int per_group = kGroupM * n_tiles;
  int group = t / per_group;
  int first_m = group * kGroupM;
  int gsz = min(m_tiles - first_m, kGroupM);
  int r = t - group * per_group;
  tm = first_m + (r % gsz);
  tn = r / gsz;
}

__device__ __forceinline__ void unit_to_tile(const GemmParams& p, int unit, int& tm, int& tn, int& split) {
  unit_to_tile_n(p.m_tiles, p.n_tiles, unit, tm, tn, split);
}

// ---------------------------------------------------------------------------------------------------------------
// Eight-warp accumulator drain shared by the dense kernels (single CTA and CTA pair).
//
// The eight epilogue warps are two groups of four. TMEM lanes [32q, 32q + 32) can only be read by a warp whose index
// is q modulo 4, so each group has one warp per lane quarter; group g takes columns [g * BN/2, (g+1) * BN/2) of the
// accumulator. A warp reads one 64-column slab of its 32 rows with two tcgen05.ld in flight under one wait (the global
// loads of the residual / saved pre-activation are issued before that wait), releases the accumulator as soon as its
// last slab sits in registers, then does the arithmetic and hands the bf16 slab to TMA:
//   staged path - the four warps of a group fill one 128-row x 64-column swizzled buffer (16 KB) and one thread
//                 stores it with a single cp.async.bulk.tensor (4 stores per 128 x 256 tile instead of 16);
//   direct path - fp32 output, split-K partials and accumulate-into-C go straight from registers to global memory.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kEpiWarps = 8;
constexpr int kDenseThreads = 64 + 32 * kEpiWarps;   // producer warp + MMA warp + epilogue warps
constexpr int kDenseStagingBytes = 2 * 16384;        // per staging buffer of each group: two groups x 128 x 64 bf16

// Which compile-time variant of the slab arithmetic a product takes (GemmParams::epi_mode); 0 keeps every test at
// run time (column scales, odd alignments, ragged column edges).
enum EpiMode : int { kEpiGeneric = 0, kEpiPlain, kEpiBias, kEpiBiasRes, kEpiRes, kEpiBiasGelu, kEpiGelu, kEpiGeluGrad,
                     kEpiBiasGeluD, kEpiGeluD, kEpiMulAux };

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// 32 columns (64 bytes: two whole sectors) of this thread's row of a row-major bf16 matrix - the residual, or the
// saved pre-activation. Rows at or past `rows` read as zero.
__device__ __forceinline__ void side_fetch(const __nv_bfloat16* base, int ld, int row, int rows, int col,
                                           uint4 (&v)[4]) {
  const uint4* src = reinterpret_cast<const uint4*>(base + size_t(row) * ld + col);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = (row < rows) ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
}

// Arithmetic of 32 full, 16-byte-aligned columns (half `half` of the slab at col0) of one row. `acc` are raw
// accumulators; `sidev` the same columns of the residual (RES) or of the saved pre-activation
// (ACT == kActGeluGrad); `out` receives packed bf16 pairs - for ACT == kActGelu the pre-activation, to which the
// caller applies gelu_of_packed after it has been stored.
template <bool BIAS, int ACT, bool RES>
__device__ __forceinline__ void half_math(const GemmParams& p, int col0, int half, const uint32_t (&acc)[32],
                                          const uint4 (&sidev)[4], uint32_t (&out)[16], uint32_t (&second)[16]) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float v[8];
    uint32_t side[4];
    if (RES || ACT == kActGeluGrad || ACT == kActMulAux) {
      side[0] = sidev[g].x; side[1] = sidev[g].y; side[2] = sidev[g].z; side[3] = sidev[g].w;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc[g * 8 + i]) * p.alpha;
    if (BIAS) {
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + half * 32 + g * 8));
      float2 f;
      f = unpack_bf16x2(b.x); v[0] += f.x; v[1] += f.y;
      f = unpack_bf16x2(b.y); v[2] += f.x; v[3] += f.y;
      f = unpack_bf16x2(b.z); v[4] += f.x; v[5] += f.y;
      f = unpack_bf16x2(b.w); v[6] += f.x; v[7] += f.y;
    }
    if (ACT == kActGeluGrad) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = unpack_bf16x2(side[i]);
        v[2 * i] *= gelu_tanh_grad(x.x);
        v[2 * i + 1] *= gelu_tanh_grad(x.y);
      }
    } else if (ACT == kActMulAux) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = unpack_bf16x2(side[i]);
        v[2 * i] *= x.x;
        v[2 * i + 1] *= x.y;
      }
    } else if (ACT == kActGeluD) {
      // value and derivative from the one tanh; `second` takes the derivative
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float g0, d0, g1, d1;
        gelu_tanh_both(v[2 * i], g0, d0);
        gelu_tanh_both(v[2 * i + 1], g1, d1);
        v[2 * i] = g0;
        v[2 * i + 1] = g1;
        second[g * 4 + i] = pack_bf16x2(d0, d1);
      }
    }
    if (RES) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(side[i]);
        v[2 * i] += f.x;
        v[2 * i + 1] += f.y;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) out[g * 4 + i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
  }
}

// GELU of packed bf16 values in place: the activation sees the value as it is stored, so forward and backward agree.
__device__ __forceinline__ void gelu_of_packed(uint32_t (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float2 f = unpack_bf16x2(v[i]);
    v[i] = pack_bf16x2(gelu_tanh(f.x), gelu_tanh(f.y));
  }
}

// Run-time-tested variant of half_math (any alignment, ragged column edge, column scales). With kActGelu `out`
// holds the activation and `pre` the pre-activation.
__device__ __forceinline__ void half_math_generic(const GemmParams& p, int row, int col0, int half,
                                                  const uint32_t (&acc)[32], uint32_t (&out)[16], uint32_t (&pre)[16]) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int col = col0 + half * 32 + g * 8;
    float v[8], pr[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] = __uint_as_float(acc[g * 8 + i]) * p.alpha; pr[i] = 0.f; }
    if (row < p.M && col < p.N) epilogue_math8(p, row, col, v, min(8, p.N - col), false, pr);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[g * 4 + i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
      pre[g * 4 + i] = pack_bf16x2(pr[2 * i], pr[2 * i + 1]);
    }
  }
}

// Write 32 packed columns (half `half` of the slab) into row `r` (0..127) of a 128-byte-swizzled 128 x 64 buffer.
__device__ __forceinline__ void half_to_smem(uint8_t* buf, int r, int half, const uint32_t* v) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 o;
    o.x = v[4 * c]; o.y = v[4 * c + 1]; o.z = v[4 * c + 2]; o.w = v[4 * c + 3];
    *reinterpret_cast<uint4*>(buf + r * 128 + (((4 * half + c) ^ (r & 7)) << 4)) = o;
  }
}

__device__ __forceinline__ bool mode_has_side(int mode) {
  return mode == kEpiBiasRes || mode == kEpiRes || mode == kEpiGeluGrad || mode == kEpiMulAux;
}
__device__ __forceinline__ bool mode_side_is_aux(int mode) { return mode == kEpiGeluGrad || mode == kEpiMulAux; }

// The side input a thread fetched ahead of the half-slab it will drain next (16 registers carried across halves,
// slabs and tiles), so the global-memory latency of the residual / saved pre-activation is off the critical path.
struct SideAhead {
  uint4 v[4];
  bool ready;       // uniform over the warp
  int ring;         // which of the group's staging buffers the next store takes (uniform over the group)
};
// The tile this CTA drains after the current one.
struct NextTile {
  bool valid;
  int row_base, n0;
};

// Drain this CTA's 128 x BN accumulator at TMEM address `acc_taddr` (lane 0, first column of the buffer).
//   ewarp      0..7, index of the calling warp among the epilogue warps (its hardware warp index must be ewarp + 2)
//   row_base   first global row of the accumulator's 128 rows, n0 its first global column
//   staging    kBufs * kDenseStagingBytes of shared memory, 1024-byte aligned: kBufs buffers per group. With two, a
//              store only waits for the one before the last to have been read, which by then it long has
//   release    called by every thread once its last tcgen05.ld has completed (arrives on the accumulator's barrier)
//   ahead/next this warp's prefetched side input and the tile it drains next
// `have_acc` false stands for a split past the end of K: zeros are drained without touching TMEM.
// The accumulator is read 32 columns at a time so the whole drain fits the 168 registers a 10-warp CTA leaves a
// thread without spilling.
template <int BN, int kBufs, typename Release>
__device__ __forceinline__ void drain_accumulator(const GemmParams& p, const CUtensorMap* tmC, const CUtensorMap* tmAux,
                                                  uint32_t acc_taddr, int ewarp, int lane, int row_base, int n0,
                                                  int split, bool have_acc, uint8_t* staging, SideAhead& ahead,
                                                  const NextTile& next, Release release) {
  constexpr int kSlabs = BN / 128;                    // 64-column slabs per group
  const int quarter = (ewarp + 2) & 3;
  const int group = ewarp >> 2;
  const int r_in_tile = quarter * 32 + lane;
  const int row = row_base + r_in_tile;
  const uint32_t lane_taddr = acc_taddr + (uint32_t(quarter * 32) << 16);
  const bool staged = p.tma_store && p.splits == 1;
  const bool leader = (quarter == 0) && (lane == 0);  // issues and waits for this group's TMA stores
  const bool gelu = (p.act == kActGelu);
  const bool two_outputs = gelu || (p.act == kActGeluD);
  bool released = false;

#pragma unroll 1
  for (int j = 0; j < kSlabs; ++j) {
    const int cslab = group * kSlabs + j;
    const int col0 = n0 + cslab * 64;
    if (col0 >= p.N) break;                           // uniform over the group
    const bool last_slab = (j == kSlabs - 1) || (col0 + 64 >= p.N);
    if (staged) {
      const int mode = (col0 + 64 <= p.N) ? p.epi_mode : kEpiGeneric;      // uniform over the warp
      const bool has_side = mode_has_side(mode);
      const __nv_bfloat16* side_base = mode_side_is_aux(mode) ? p.aux : p.residual;
      const int side_ld = mode_side_is_aux(mode) ? p.ld_aux : p.ldr;
      uint32_t out[32];                               // the slab's packed output (kActGelu: its pre-activation)
      uint32_t second[32];                            // what goes to aux: generic GELU's pre-activation, kActGeluD's derivative
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t acc[32];
        if (have_acc) {
          tmem_ld_32x32b_x32(lane_taddr + cslab * 64 + h * 32, acc);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = 0u;
        }
        uint4 cur[4];
        if (has_side) {
          if (ahead.ready) {
#pragma unroll
            for (int i = 0; i < 4; ++i) cur[i] = ahead.v[i];
          } else {
            side_fetch(side_base, side_ld, row, p.M, col0 + h * 32, cur);
          }
          ahead.ready = false;
          // fetch ahead: the other half of this slab, else the first half of the slab this warp drains next
          int nrow = -1, ncol = 0;
          if (h == 0) { nrow = row; ncol = col0 + 32; }
          else if (!last_slab) { nrow = row; ncol = col0 + 64; }
          else if (next.valid && next.n0 + group * kSlabs * 64 + 64 <= p.N) {
            nrow = next.row_base + r_in_tile;
            ncol = next.n0 + group * kSlabs * 64;
          }
          if (nrow >= 0 && (h == 0 || ncol + 64 <= p.N)) {
            side_fetch(side_base, side_ld, nrow, p.M, ncol, ahead.v);
            ahead.ready = true;
          }
        }
        if (have_acc) tmem_ld_wait();
        if (h == 1 && last_slab) { release(); released = true; }
        uint32_t(&o)[16] = *reinterpret_cast<uint32_t(*)[16]>(&out[h * 16]);
        uint32_t(&o2)[16] = *reinterpret_cast<uint32_t(*)[16]>(&second[h * 16]);
        switch (mode) {
          case kEpiPlain:     half_math<false, kActNone, false>(p, col0, h, acc, cur, o, o2); break;
          case kEpiBias:      half_math<true, kActNone, false>(p, col0, h, acc, cur, o, o2); break;
          case kEpiBiasRes:   half_math<true, kActNone, true>(p, col0, h, acc, cur, o, o2); break;
          case kEpiRes:       half_math<false, kActNone, true>(p, col0, h, acc, cur, o, o2); break;
          case kEpiBiasGelu:  half_math<true, kActGelu, false>(p, col0, h, acc, cur, o, o2); break;
          case kEpiGelu:      half_math<false, kActGelu, false>(p, col0, h, acc, cur, o, o2); break;
          case kEpiGeluGrad:  half_math<false, kActGeluGrad, false>(p, col0, h, acc, cur, o, o2); break;
          case kEpiBiasGeluD: half_math<true, kActGeluD, false>(p, col0, h, acc, cur, o, o2); break;
          case kEpiGeluD:     half_math<false, kActGeluD, false>(p, col0, h, acc, cur, o, o2); break;
          case kEpiMulAux:    half_math<false, kActMulAux, false>(p, col0, h, acc, cur, o, o2); break;
          default:            half_math_generic(p, row, col0, h, acc, o, o2); break;
        }
      }
      // registers -> this group's next staging buffer -> one TMA store of the 128 x 64 slab
      auto stage_and_store = [&](const CUtensorMap* tm, const uint32_t* vals) {
        uint8_t* b = staging + (group * kBufs + ahead.ring) * 16384;
        if (leader) tma_store_wait_read<kBufs - 1>();   // the store that last used this buffer has read it
        named_bar_sync(1 + group, 128);
        half_to_smem(b, r_in_tile, 0, vals);
        half_to_smem(b, r_in_tile, 1, vals + 16);
        fence_proxy_async_smem();
        named_bar_sync(1 + group, 128);
        if (leader) {
          tma_store_2d(tm, b, col0, row_base);
          tma_store_commit();
        }
        ahead.ring = (ahead.ring + 1) % kBufs;
      };
      if (two_outputs) {
        // what is saved for the backward pass leaves first. kActGelu: the pre-activation, and the activation is
        // evaluated while that store reads the buffer; kActGeluD and the generic path hold both outputs already
        const bool pre_in_out = gelu && mode != kEpiGeneric;
        stage_and_store(tmAux, pre_in_out ? out : second);
        if (pre_in_out) gelu_of_packed(out);
      }
      stage_and_store(tmC, out);
    } else {
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t acc[32];
        if (have_acc) {
          tmem_ld_32x32b_x32(lane_taddr + cslab * 64 + h * 32, acc);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = 0u;
        }
        if (h == 1 && last_slab) { release(); released = true; }
        const int c32 = col0 + h * 32;
        if (row < p.M && c32 < p.N) {
          if (p.splits > 1) {
            float* w = p.workspace + (size_t(split) * p.M + row) * p.N + c32;
            if (c32 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(w) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(w)[i] =
                    make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                                __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
            } else {
              for (int i = 0; i < 32 && c32 + i < p.N; ++i) w[i] = __uint_as_float(acc[i]);
            }
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = c32 + g * 8;
              if (col < p.N) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc[g * 8 + i]) * p.alpha;
                epilogue8(p, row, col, v, min(8, p.N - col));
              }
            }
          }
        }
      }
    }
  }
  if (!released) release();
}

// Host side: the staged epilogue's compile-time variant for a filled parameter block, and the role-timer buffer
// (null unless idrak_gemm_role_timers switched it on).
int pick_epi_mode(const GemmParams& p);
unsigned long long* role_timer_buffer();
// The CTA-pair kernel (gemm2_tcgen05.cu): whether a product should use it, and its launcher.
bool gemm_pair_wanted(int M, int N, int K, int splits);
int gemm_pair_launch(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, const CUtensorMap& tmC,
                     const CUtensorMap& tmAux, GemmParams p, int fp16, cudaStream_t stream);
}  // namespace idrak
