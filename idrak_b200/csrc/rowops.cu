// Row-wise and element-wise kernels on bf16 activations: LayerNorm / RMSNorm forward and backward,
// GELU, gated activations (SwiGLU family), RoPE, embedding lookup and its gradients, column sums
// (bias gradients) and dtype conversion. All are bandwidth-bound: 128-bit loads and stores, one warp
// per row with the row held in registers where it fits, fp32 arithmetic, fixed-order reductions (no
// float atomics) so reruns give the same bits.
//
// Reference counterparts: rms_norm_f32 / rms_norm_backward_f32 / rope_f32 / gated_act_f32(+bwd)
// (src/Idrak.Gpu/Cuda/PtxKernels.Decoder.cs:14), layernorm_train_f32 / layernorm_bwd_f32 /
// layernorm_bwd_params_f32 / bias_gelu_f32 (PtxKernels.Decoding.cs:12), gather / scatter and
// sum_cols_strided (PtxKernels.Advanced.cs:12, PtxKernels.Rows.cs:13).
#include "common.cuh"
#include "norm_bulk.h"
#include <cstdlib>

namespace idrak {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 a = *reinterpret_cast<const uint4*>(p);
  float2 f;
  f = unpack_bf16x2(a.x); v[0] = f.x; v[1] = f.y;
  f = unpack_bf16x2(a.y); v[2] = f.x; v[3] = f.y;
  f = unpack_bf16x2(a.z); v[4] = f.x; v[5] = f.y;
  f = unpack_bf16x2(a.w); v[6] = f.x; v[7] = f.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// ---------------------------------------------------------------------------
// LayerNorm / RMSNorm forward. One warp per row; C % 8 == 0; row cached in registers for C <= 8*32*VPL.
// `rms` = 1 selects RMSNorm (no mean subtraction, no bias).
// Optional `residual`: the row normalised is x + residual and that sum is written to `sum_out`.
// ---------------------------------------------------------------------------
template <int VPL>
__global__ void __launch_bounds__(128) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                       const __nv_bfloat16* __restrict__ residual,
                                                       const __nv_bfloat16* __restrict__ w,
                                                       const __nv_bfloat16* __restrict__ b,
                                                       __nv_bfloat16* __restrict__ out,
                                                       __nv_bfloat16* __restrict__ sum_out,
                                                       float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                       int rows, int C, float eps, int rms) {
  pdl_launch_dependents();     // a dependent launched programmatically may set itself up while this kernel runs
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const size_t base = size_t(warp) * C;
  const int nvec = C >> 3;
  float v[VPL][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      load8(x + base + vi * 8, v[i]);
      if (residual) {
        float r[8];
        load8(residual + base + vi * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        if (sum_out) {
          store8(sum_out + base + vi * 8, v[i]);
          // normalise what was stored, so a later backward pass that re-reads the sum sees the same input
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
  }
  float mean = 0.f;
  if (!rms) mean = warp_sum(s) / float(C);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float d = v[i][j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / float(C) + eps);
  if (lane == 0) {
    if (mean_out) mean_out[warp] = mean;
    if (rstd_out) rstd_out[warp] = rstd;
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      float wv[8], bv[8], o[8];
      load8(w + vi * 8, wv);
      if (b) load8(b + vi * 8, bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float n = (v[i][j] - mean) * rstd;
        o[j] = n * wv[j] + (b ? bv[j] : 0.f);
      }
      store8(out + base + vi * 8, o);
    }
  }
}

// The same forward for a handful of long rows (a decode step): one 256-thread block per row, so a row's loads
// are spread over eight warps instead of queueing behind one. C % 8 == 0, C <= 8 * 256 * 4.
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();                       // red may still be read from the previous call
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}

__global__ void __launch_bounds__(256) norm_fwd_block_kernel(const __nv_bfloat16* __restrict__ x,
                                                             const __nv_bfloat16* __restrict__ residual,
                                                             const __nv_bfloat16* __restrict__ w,
                                                             const __nv_bfloat16* __restrict__ b,
                                                             __nv_bfloat16* __restrict__ out,
                                                             __nv_bfloat16* __restrict__ sum_out,
                                                             float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                             int rows, int C, float eps, int rms) {
  pdl_launch_dependents();     // a dependent launched programmatically may set itself up while this kernel runs
  __shared__ float red[8];
  const int row = blockIdx.x;
  const size_t base = size_t(row) * C;
  const int nvec = C >> 3;
  float v[4][8], wv[4][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      load8(x + base + vi * 8, v[i]);
      load8(w + vi * 8, wv[i]);
      if (residual) {
        float r[8];
        load8(residual + base + vi * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        if (sum_out) {
          store8(sum_out + base + vi * 8, v[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
  }
  float mean = 0.f;
  if (!rms) mean = block_sum_256(s, red) / float(C);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (threadIdx.x + i * 256 < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[i][j] - mean;
        q += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum_256(q, red) / float(C) + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      float bv[8], o[8];
      if (b) load8(b + vi * 8, bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * wv[i][j] + (b ? bv[j] : 0.f);
      store8(out + base + vi * 8, o);
    }
  }
}

// ---------------------------------------------------------------------------
// LayerNorm / RMSNorm backward. One warp per row for dx; each block also accumulates the rows it owns
// into per-block partial sums of dw / db ([gridDim.x, C] fp32) which `colsum_final_kernel` folds in
// block order. `dres_in` (optional) is added to dx: the gradient arriving through the residual path.
// ---------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(128) norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                       const __nv_bfloat16* __restrict__ x,
                                                       const __nv_bfloat16* __restrict__ w,
                                                       const float* __restrict__ mean_in,
                                                       const float* __restrict__ rstd_in,
                                                       const __nv_bfloat16* __restrict__ dres_in,
                                                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part,
                                                       float* __restrict__ db_part, int rows, int C, int rms,
                                                       int rows_per_block) {
  // A block walks its rows one after another; each thread owns fixed columns (vectors tid + i*128), so
  // the dw / db partial sums stay in registers and are added in row order.
  __shared__ float red[2][4];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int nvec = C >> 3;
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  float adw[VPT][8], adb[VPT][8], wv[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = tid + i * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j) { adw[i][j] = 0.f; adb[i][j] = 0.f; wv[i][j] = 0.f; }
    if (vi < nvec) load8(w + vi * 8, wv[i]);
  }
  for (int row = row0; row < row1; ++row) {
    const size_t base = size_t(row) * C;
    const float mean = rms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float g[VPT][8], n[VPT][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tid + i * 128;
      if (vi < nvec) {
        float dyv[8], xv[8];
        load8(dy + base + vi * 8, dyv);
        load8(x + base + vi * 8, xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          n[i][j] = (xv[j] - mean) * rstd;
          g[i][j] = dyv[j] * wv[i][j];
          s1 += g[i][j];
          s2 += g[i][j] * n[i][j];
          adw[i][j] += dyv[j] * n[i][j];
          adb[i][j] += dyv[j];
        }
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    __syncthreads();   // the previous row's readers are done with `red`
    if (lane == 0) { red[0][wid] = s1; red[1][wid] = s2; }
    __syncthreads();
    s1 = rms ? 0.f : (red[0][0] + red[0][1] + red[0][2] + red[0][3]) / float(C);
    s2 = (red[1][0] + red[1][1] + red[1][2] + red[1][3]) / float(C);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = tid + i * 128;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (g[i][j] - s1 - n[i][j] * s2) * rstd;
        if (dres_in) {
          float r[8];
          load8(dres_in + base + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + base + vi * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = tid + i * 128;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dw_part[size_t(blockIdx.x) * C + vi * 8 + j] = adw[i][j];
        if (db_part) db_part[size_t(blockIdx.x) * C + vi * 8 + j] = adb[i][j];
      }
    }
  }
}

// out[c] (+)= sum_p part[p, c]. Block = 32 columns x 8 part lanes: lane ty adds parts ty, ty+8, ... in
// ascending order, then the 8 lane sums are added in lane order, so the result has one fixed order.
__global__ void __launch_bounds__(256) colsum_final_kernel(const float* __restrict__ part, int parts, int C,
                                                           void* __restrict__ out, int out_fp32, int accumulate) {
  __shared__ float sm[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < C)
    for (int p = ty; p < parts; p += 8) s += part[size_t(p) * C + c];
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < C) {
    float r = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) r += sm[k][tx];
    if (out_fp32) {
      float* o = static_cast<float*>(out);
      o[c] = accumulate ? o[c] + r : r;
    } else {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
      o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + r : r);
    }
  }
}

// Column sums of a bf16 matrix [rows, C] (ld elements per row) into per-block partials [gridDim.y, C].
// Block = 32 x 8 threads: a lane owns 8 consecutive columns (one 128-bit load per row), 8 row lanes stride
// the rows of the block's chunk. Needs ld % 8 == 0 and a 16-byte aligned base; C may be ragged.
__global__ void __launch_bounds__(256) colsum_part_kernel(const __nv_bfloat16* __restrict__ x, int rows, int C,
                                                          int ld, int rows_per_block, float* __restrict__ part) {
  __shared__ float sm[8][256];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + tx * 8;
  const int row0 = blockIdx.y * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  float a[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = 0.f;
  if (col + 8 <= C) {
    for (int r = row0 + ty; r < row1; r += 8) {
      float v[8];
      load8(x + size_t(r) * ld + col, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += v[j];
    }
  } else if (col < C) {
    for (int r = row0 + ty; r < row1; r += 8)
      for (int j = 0; j < C - col; ++j) a[j] += __bfloat162float(x[size_t(r) * ld + col + j]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[ty][tx * 8 + j] = a[j];
  __syncthreads();
  const int c = threadIdx.x;          // 256 threads fold the 256 columns of the block
  if (blockIdx.x * 256 + c < C) {
    float r = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) r += sm[k][c];
    part[size_t(blockIdx.y) * C + blockIdx.x * 256 + c] = r;
  }
}

// Same contract for matrices whose rows are not 16-byte aligned: two columns per lane, scalar loads.
__global__ void __launch_bounds__(256) colsum_part_scalar_kernel(const __nv_bfloat16* __restrict__ x, int rows,
                                                                 int C, int ld, int rows_per_block,
                                                                 float* __restrict__ part) {
  __shared__ float sm[8][64];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + tx * 2;
  const int row0 = blockIdx.y * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  float a0 = 0.f, a1 = 0.f;
  if (col < C) {
    for (int r = row0 + ty; r < row1; r += 8) {
      const __nv_bfloat16* p = x + size_t(r) * ld + col;
      a0 += __bfloat162float(p[0]);
      if (col + 1 < C) a1 += __bfloat162float(p[1]);
    }
  }
  sm[ty][tx * 2] = a0;
  sm[ty][tx * 2 + 1] = a1;
  __syncthreads();
  if (ty == 0) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { s0 += sm[k][tx * 2]; s1 += sm[k][tx * 2 + 1]; }
    if (col < C) part[size_t(blockIdx.y) * C + col] = s0;
    if (col + 1 < C) part[size_t(blockIdx.y) * C + col + 1] = s1;
  }
}

// LayerNorm / RMSNorm backward for rows that fit a warp's registers (C <= 256 * VPL): one warp per row, eight
// warps per block walking the block's rows; per-lane dw / db sums are folded across the warps of a block in
// warp order through shared memory, so the per-block partials have a fixed summation order.
template <int VPL>
__global__ void __launch_bounds__(256, 2) norm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy,
                                                            const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            const float* __restrict__ mean_in,
                                                            const float* __restrict__ rstd_in,
                                                            const __nv_bfloat16* __restrict__ dres_in,
                                                            __nv_bfloat16* __restrict__ dx,
                                                            float* __restrict__ dw_part, float* __restrict__ db_part,
                                                            int rows, int C, int rms, int rows_per_block) {
  extern __shared__ float sm_acc[];   // [2][C]
  float* sdw = sm_acc;
  float* sdb = sm_acc + C;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  float adw[VPL][8], adb[VPL][8], wv[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
#pragma unroll
    for (int j = 0; j < 8; ++j) { adw[i][j] = 0.f; adb[i][j] = 0.f; wv[i][j] = 0.f; }
    if (vi < nvec) load8(w + vi * 8, wv[i]);
  }
  for (int row = row0 + wid; row < row1; row += 8) {
    const size_t base = size_t(row) * C;
    const float mean = rms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float g[VPL][8], n[VPL][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float dyv[8], xv[8];
        load8(dy + base + vi * 8, dyv);
        load8(x + base + vi * 8, xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          n[i][j] = (xv[j] - mean) * rstd;
          g[i][j] = dyv[j] * wv[i][j];
          s1 += g[i][j];
          s2 += g[i][j] * n[i][j];
          adw[i][j] += dyv[j] * n[i][j];
          adb[i][j] += dyv[j];
        }
      }
    }
    s1 = rms ? 0.f : warp_sum(s1) / float(C);
    s2 = warp_sum(s2) / float(C);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (g[i][j] - s1 - n[i][j] * s2) * rstd;
        if (dres_in) {
          float r[8];
          load8(dres_in + base + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + base + vi * 8, o);
      }
    }
  }
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) sm_acc[i] = 0.f;
  __syncthreads();
  for (int wsel = 0; wsel < 8; ++wsel) {
    if (wid == wsel) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int vi = lane + i * 32;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            sdw[vi * 8 + j] += adw[i][j];
            sdb[vi * 8 + j] += adb[i][j];
          }
        }
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    dw_part[size_t(blockIdx.x) * C + i] = sdw[i];
    if (db_part) db_part[size_t(blockIdx.x) * C + i] = sdb[i];
  }
}

// ---------------------------------------------------------------------------
// element-wise: GELU (tanh form), gated activations, add, scale, convert
// ---------------------------------------------------------------------------
enum { kGateSilu = 0, kGateGelu = 1, kGateRelu = 2, kGateTanh = 3 };

__device__ __forceinline__ float gate_fn(float g, int kind) {
  switch (kind) {
    case kGateSilu: return g / (1.f + __expf(-g));
    case kGateGelu: return gelu_tanh(g);
    case kGateRelu: return fmaxf(g, 0.f);
    default: return tanhf(g);
  }
}
__device__ __forceinline__ float gate_grad(float g, int kind) {
  switch (kind) {
    case kGateSilu: {
      float s = 1.f / (1.f + __expf(-g));
      return s * (1.f + g * (1.f - s));
    }
    case kGateGelu: return gelu_tanh_grad(g);
    case kGateRelu: return g > 0.f ? 1.f : 0.f;
    default: {
      float t = tanhf(g);
      return 1.f - t * t;
    }
  }
}

__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n8) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n8; i += size_t(gridDim.x) * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
    store8(y + i * 8, v);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, size_t n8) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n8; i += size_t(gridDim.x) * blockDim.x) {
    float v[8], g[8];
    load8(x + i * 8, v);
    load8(dy + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= gelu_tanh_grad(v[j]);
    store8(dx + i * 8, g);
  }
}

// gate_up: [rows, 2*H] with gate in columns [0,H) and up in [H,2H); out[r, h] = act(gate) * up.
__global__ void gated_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int rows,
                                 int H, int kind) {
  pdl_launch_dependents();     // a dependent launched programmatically may set itself up while this kernel runs
  const int hv = H >> 3;
  const size_t total = size_t(rows) * hv;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / hv;
    const int c = int(i - r * hv) * 8;
    float g[8], u[8];
    load8(gu + r * 2 * H + c, g);
    load8(gu + r * 2 * H + H + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = gate_fn(g[j], kind) * u[j];
    store8(out + r * H + c, g);
  }
}
__global__ void gated_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                 __nv_bfloat16* __restrict__ dgu, int rows, int H, int kind) {
  const int hv = H >> 3;
  const size_t total = size_t(rows) * hv;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / hv;
    const int c = int(i - r * hv) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + r * 2 * H + c, g);
    load8(gu + r * 2 * H + H + c, u);
    load8(dout + r * H + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * u[j] * gate_grad(g[j], kind);
      du[j] = d[j] * gate_fn(g[j], kind);
    }
    store8(dgu + r * 2 * H + c, dg);
    store8(dgu + r * 2 * H + H + c, du);
  }
}

__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ y, size_t n8) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n8; i += size_t(gridDim.x) * blockDim.x) {
    float u[8], v[8];
    load8(a + i * 8, u);
    load8(b + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] += v[j];
    store8(y + i * 8, u);
  }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n) {
  for (size_t i = (blockIdx.x * size_t(blockDim.x) + threadIdx.x) * 4; i < n;
       i += size_t(gridDim.x) * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 v = *reinterpret_cast<const float4*>(x + i);
      uint2 o;
      o.x = pack_bf16x2(v.x, v.y);
      o.y = pack_bf16x2(v.z, v.w);
      *reinterpret_cast<uint2*>(y + i) = o;
    } else {
      for (size_t j = i; j < n; ++j) y[j] = __float2bfloat16(x[j]);
    }
  }
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, size_t n) {
  for (size_t i = (blockIdx.x * size_t(blockDim.x) + threadIdx.x) * 4; i < n;
       i += size_t(gridDim.x) * blockDim.x * 4) {
    if (i + 4 <= n) {
      uint2 a = *reinterpret_cast<const uint2*>(x + i);
      float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y);
      *reinterpret_cast<float4*>(y + i) = make_float4(f0.x, f0.y, f1.x, f1.y);
    } else {
      for (size_t j = i; j < n; ++j) y[j] = __bfloat162float(x[j]);
    }
  }
}

// ---------------------------------------------------------------------------
// RoPE on [tokens, heads, head_dim] in place. Rotate-half convention (pairs (i, i + D/2)), the one
// Llama-family checkpoints in Hugging Face layout use. positions[t] gives the absolute position.
// inverse = 1 applies the transposed rotation (the backward pass).
// ---------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ positions, int tokens, int heads,
                            int D, int row_stride, int rot_dim, float theta, float freq_scale, int inverse) {
  const int half = rot_dim >> 1;
  const size_t total = size_t(tokens) * heads * half;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const int k = int(i % half);
    const size_t th = i / half;
    const int h = int(th % heads);
    const size_t t = th / heads;
    const float pos = float(positions ? positions[t] : int(t)) * freq_scale;
    const float inv_freq = __powf(theta, -2.0f * float(k) / float(rot_dim));
    float s, c;
    sincosf(pos * inv_freq, &s, &c);
    if (inverse) s = -s;
    __nv_bfloat16* p = x + t * row_stride + size_t(h) * D;
    const float a = __bfloat162float(p[k]), b = __bfloat162float(p[k + half]);
    p[k] = __float2bfloat16(a * c - b * s);
    p[k + half] = __float2bfloat16(b * c + a * s);
  }
}

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = wte[ids[t], :] (+ wpe[t % seq, :]).
// ---------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out,
                                     int tokens, int seq, int C) {
  const int cv = C >> 3;
  const size_t total = size_t(tokens) * cv;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t t = i / cv;
    const int c = int(i - t * cv) * 8;
    float v[8];
    load8(wte + size_t(ids[t]) * C + c, v);
    if (wpe) {
      float p[8];
      load8(wpe + size_t(t % seq) * C + c, p);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += p[j];
    }
    store8(out + t * C + c, v);
  }
}

// Position-table gradient: dwpe[s, :] (+)= sum_b dout[b*seq + s, :], b ascending.
__global__ void wpe_bwd_kernel(const __nv_bfloat16* __restrict__ dout, void* __restrict__ dwpe, int batch, int seq,
                               int C, int out_fp32, int accumulate) {
  const int cv = C >> 3;
  const size_t total = size_t(seq) * cv;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t s = i / cv;
    const int c = int(i - s * cv) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int b = 0; b < batch; ++b) {
      float v[8];
      load8(dout + (size_t(b) * seq + s) * C + c, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
    if (out_fp32) {
      float* o = static_cast<float*>(dwpe) + s * C + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = accumulate ? o[j] + acc[j] : acc[j];
    } else {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(dwpe) + s * C + c;
      if (accumulate) {
        float old[8];
        load8(o, old);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += old[j];
      }
      store8(o, acc);
    }
  }
}

// Token-table gradient from tokens sorted by id: `order` lists token positions so that ids[order[i]] is
// non-decreasing. One block per run of equal ids adds its rows in `order` sequence (stable sort =>
// ascending token position), then adds into dwte (which may already hold the tied head's gradient).
__global__ void wte_bwd_kernel(const int* __restrict__ sorted_ids, const int* __restrict__ order,
                               const __nv_bfloat16* __restrict__ dout, void* __restrict__ dwte, int tokens, int C,
                               int out_fp32) {
  const int i0 = blockIdx.x;
  if (i0 >= tokens) return;
  const int id = sorted_ids[i0];
  if (i0 > 0 && sorted_ids[i0 - 1] == id) return;   // not the first of its run
  const int cv = C >> 3;
  for (int v = threadIdx.x; v < cv; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int i = i0; i < tokens && sorted_ids[i] == id; ++i) {
      float g[8];
      load8(dout + size_t(order[i]) * C + v * 8, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += g[j];
    }
    if (out_fp32) {
      float* o = static_cast<float*>(dwte) + size_t(id) * C + v * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] += acc[j];
    } else {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(dwte) + size_t(id) * C + v * 8;
      float old[8];
      load8(o, old);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += old[j];
      store8(o, acc);
    }
  }
}

static inline int grid_for(size_t work, int block, int cap_per_sm = 8) {
  size_t g = (work + block - 1) / block;
  size_t cap = size_t(sm_count()) * cap_per_sm;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace idrak

using namespace idrak;

#define BF(p) static_cast<__nv_bfloat16*>(p)
#define CBF(p) static_cast<const __nv_bfloat16*>(p)

// LayerNorm (rms=0) / RMSNorm (rms=1) forward. C % 8 == 0 and C <= 8192.
IDRAK_API int idrak_norm_fwd(const void* x, const void* residual, const void* w, const void* b, void* out,
                             void* sum_out, float* mean, float* rstd, int rows, int C, float eps, int rms,
                             void* stream_) {
  if (C % 8 || C > 8192 || rows <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int blocks = (rows + 3) / 4;
  const int nvec = C / 8;
  if (rows <= 2 * sm_count() && nvec >= 128) {      // few long rows: a block per row
    norm_fwd_block_kernel<<<rows, 256, 0, s>>>(CBF(x), CBF(residual), CBF(w), CBF(b), BF(out), BF(sum_out), mean, rstd,
                                               rows, C, eps, rms);
    note_launches(1);
    return int(cudaGetLastError());
  }
#define NF(V) norm_fwd_kernel<V><<<blocks, 128, 0, s>>>(CBF(x), CBF(residual), CBF(w), CBF(b), BF(out), BF(sum_out), mean, rstd, rows, C, eps, rms)
  if (nvec <= 32 * 1) NF(1);
  else if (nvec <= 32 * 2) NF(2);
  else if (nvec <= 32 * 4) NF(4);
  else if (nvec <= 32 * 8) NF(8);
  else if (nvec <= 32 * 16) NF(16);
  else NF(32);
#undef NF
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_colsum(const void* x, int rows, int C, int ld, float* part, void* out, int out_fp32,
                           int accumulate, void* stream_);

// Number of row blocks the backward pass uses at most; its scratch holds 3 x [that, C] floats.
IDRAK_API int idrak_norm_bwd_blocks(int rows) {
  int b = sm_count() * 2;
  return rows < b ? rows : b;
}

// Backward of LayerNorm / RMSNorm. dx = norm backward of dy (+ dres_in); dw / db are written (or accumulated into)
// in fp32 or bf16. `part` holds 3 * idrak_norm_bwd_blocks(rows) * C floats. `dx_colsum` (fp32 [C], optional) receives
// the column sums of dx: the bias gradient of the linear layer whose output this norm read. Rows of up to 1024
// elements take the bulk-copy pipeline of norm_bulk.cu, which produces that sum for free; wider rows take the
// register kernels and, when the sum is asked for, a column-sum pass over dx.
IDRAK_API int idrak_norm_bwd_fused(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                   const void* dres_in, void* dx, float* part, void* dw, void* db, float* dx_colsum,
                                   int grads_fp32, int accumulate, int rows, int C, int rms, void* stream_) {
  if (C % 8 || C > 8192 || rows <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  int blocks = norm_bwd_bulk_blocks(rows, C);
  static int use_bulk = -1;
  if (use_bulk < 0) {
    const char* e = getenv("IDRAK_NORM_BULK");
    use_bulk = (e && e[0] == '0') ? 0 : 1;
  }
  if (!use_bulk) blocks = 0;
  float* dw_part = part;
  float* db_part;
  float* dxs_part;
  int rc;
  if (blocks > 0) {
    db_part = part + size_t(blocks) * C;
    dxs_part = part + size_t(2) * blocks * C;
    NormBulkParams q{};
    q.dy = CBF(dy); q.x = CBF(x); q.w = CBF(w); q.mean = mean; q.rstd = rstd; q.dres = CBF(dres_in);
    q.dx = BF(dx); q.dw_part = dw_part; q.db_part = rms ? nullptr : db_part;
    q.dxs_part = dx_colsum ? dxs_part : nullptr;
    q.rows = rows; q.C = C; q.rms = rms;
    rc = norm_bwd_bulk_launch(q, blocks, s);
    if (rc) return rc;
    if (dx_colsum) {
      colsum_final_kernel<<<(C + 31) / 32, 256, 0, s>>>(dxs_part, blocks, C, dx_colsum, 1, 0);
      note_launches(1);
    }
  } else {
    blocks = idrak_norm_bwd_blocks(rows);
    db_part = part + size_t(blocks) * C;
    const int rpb = (rows + blocks - 1) / blocks;
    const int nvec = C / 8;
#define NW(V) norm_bwd_warp_kernel<V><<<blocks, 256, size_t(2) * C * sizeof(float), s>>>(CBF(dy), CBF(x), CBF(w), mean, rstd, CBF(dres_in), BF(dx), dw_part, rms ? nullptr : db_part, rows, C, rms, rpb)
#define NB(V) norm_bwd_kernel<V><<<blocks, 128, 0, s>>>(CBF(dy), CBF(x), CBF(w), mean, rstd, CBF(dres_in), BF(dx), dw_part, rms ? nullptr : db_part, rows, C, rms, rpb)
    if (nvec <= 32 * 1) NW(1);
    else if (nvec <= 32 * 2) NW(2);
    else if (nvec <= 32 * 3) NW(3);
    else if (nvec <= 32 * 4) NW(4);
    else if (nvec <= 128 * 2) NB(2);
    else if (nvec <= 128 * 4) NB(4);
    else NB(8);
#undef NW
#undef NB
    note_launches(1);
    rc = int(cudaGetLastError());
    if (rc) return rc;
    if (dx_colsum) {
      rc = idrak_colsum(dx, rows, C, C, part + size_t(2) * blocks * C, dx_colsum, 1, 0, stream_);
      if (rc) return rc;
    }
  }
  colsum_final_kernel<<<(C + 31) / 32, 256, 0, s>>>(dw_part, blocks, C, dw, grads_fp32, accumulate);
  note_launches(1);
  if (!rms && db) {
    colsum_final_kernel<<<(C + 31) / 32, 256, 0, s>>>(db_part, blocks, C, db, grads_fp32, accumulate);
    note_launches(1);
  }
  return int(cudaGetLastError());
}

// Whether a call of these sizes gets the column sums of dx without a pass of their own (1) or not (0).
IDRAK_API int idrak_norm_bwd_sums_dx(int rows, int C) { return norm_bwd_bulk_blocks(rows, C) > 0 ? 1 : 0; }

// The same without the column sums of dx; `dw_part` and `db_part` are the two halves of one 2 * blocks * C scratch.
IDRAK_API int idrak_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                             const void* dres_in, void* dx, float* dw_part, float* db_part, void* dw, void* db,
                             int grads_fp32, int accumulate, int rows, int C, int rms, void* stream_) {
  (void)db_part;
  return idrak_norm_bwd_fused(dy, x, w, mean, rstd, dres_in, dx, dw_part, dw, db, nullptr, grads_fp32, accumulate, rows,
                              C, rms, stream_);
}

IDRAK_API int idrak_colsum_blocks(int rows) {
  int b = (rows + 63) / 64;
  return b < 1 ? 1 : (b > 128 ? 128 : b);
}

// out[c] (+)= sum_r x[r, c]; `part` holds [idrak_colsum_blocks(rows), C] floats.
IDRAK_API int idrak_colsum(const void* x, int rows, int C, int ld, float* part, void* out, int out_fp32,
                           int accumulate, void* stream_) {
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int yb = idrak_colsum_blocks(rows);
  const int rpb = (rows + yb - 1) / yb;
  if ((ld % 8) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    dim3 grid((C + 255) / 256, yb);
    colsum_part_kernel<<<grid, 256, 0, s>>>(CBF(x), rows, C, ld, rpb, part);
  } else {
    dim3 grid((C + 63) / 64, yb);
    colsum_part_scalar_kernel<<<grid, 256, 0, s>>>(CBF(x), rows, C, ld, rpb, part);
  }
  note_launches(1);
  colsum_final_kernel<<<(C + 31) / 32, 256, 0, s>>>(part, yb, C, out, out_fp32, accumulate);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_gelu_fwd(const void* x, void* y, long long n, void* stream_) {
  if (n % 8) return -2;
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(CBF(x), BF(y), n / 8);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_gelu_bwd(const void* x, const void* dy, void* dx, long long n, void* stream_) {
  if (n % 8) return -2;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(CBF(x), CBF(dy), BF(dx),
                                                                                       n / 8);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_gated_fwd(const void* gu, void* out, int rows, int H, int kind, void* stream_) {
  if (H % 8) return -2;
  gated_fwd_kernel<<<grid_for(size_t(rows) * (H / 8), 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      CBF(gu), BF(out), rows, H, kind);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_gated_bwd(const void* gu, const void* dout, void* dgu, int rows, int H, int kind,
                              void* stream_) {
  if (H % 8) return -2;
  gated_bwd_kernel<<<grid_for(size_t(rows) * (H / 8), 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      CBF(gu), CBF(dout), BF(dgu), rows, H, kind);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_add(const void* a, const void* b, void* y, long long n, void* stream_) {
  if (n % 8) return -2;
  add_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(CBF(a), CBF(b), BF(y), n / 8);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_f32_to_bf16(const float* x, void* y, long long n, void* stream_) {
  f32_to_bf16_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(x, BF(y), n);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_bf16_to_f32(const void* x, float* y, long long n, void* stream_) {
  bf16_to_f32_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(CBF(x), y, n);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_rope(void* x, const int* positions, int tokens, int heads, int D, int row_stride, int rot_dim,
                         float theta, float freq_scale, int inverse, void* stream_) {
  if (rot_dim % 2 || rot_dim > D) return -2;
  rope_kernel<<<grid_for(size_t(tokens) * heads * (rot_dim / 2), 256), 256, 0,
                static_cast<cudaStream_t>(stream_)>>>(BF(x), positions, tokens, heads, D, row_stride, rot_dim, theta,
                                                     freq_scale, inverse);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_embedding_fwd(const int* ids, const void* wte, const void* wpe, void* out, int tokens, int seq,
                                  int C, void* stream_) {
  if (C % 8) return -2;
  embedding_fwd_kernel<<<grid_for(size_t(tokens) * (C / 8), 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      ids, CBF(wte), CBF(wpe), BF(out), tokens, seq, C);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_wpe_bwd(const void* dout, void* dwpe, int batch, int seq, int C, int out_fp32, int accumulate,
                            void* stream_) {
  if (C % 8) return -2;
  wpe_bwd_kernel<<<grid_for(size_t(seq) * (C / 8), 128), 128, 0, static_cast<cudaStream_t>(stream_)>>>(
      CBF(dout), dwpe, batch, seq, C, out_fp32, accumulate);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_wte_bwd(const int* sorted_ids, const int* order, const void* dout, void* dwte, int tokens, int C,
                            int out_fp32, void* stream_) {
  if (C % 8) return -2;
  int threads = C / 8 < 128 ? ((C / 8 + 31) / 32) * 32 : 128;
  wte_bwd_kernel<<<tokens, threads, 0, static_cast<cudaStream_t>(stream_)>>>(sorted_ids, order, CBF(dout), dwte,
                                                                            tokens, C, out_fp32);
  note_launches(1);
  return int(cudaGetLastError());
}
