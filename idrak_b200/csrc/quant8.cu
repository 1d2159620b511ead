// Quantisers for the 8-bit (fp8 e4m3) tensor-core GEMM: a bf16 matrix becomes e4m3 codes plus one fp32 scale per
// row, scale = max|row| / 448 (448 is the largest finite e4m3 value), code = round-to-nearest(x / scale) with
// saturation. A GEMM over two such operands multiplies the accumulator by rowscale_A[m] * rowscale_B[n] in its
// epilogue. Both operands of the GEMM are K-major, so "per row" is per output row for activations [M, K] and per
// output column for weights stored [N, K].
//
// One warp per row: the row is read once into registers when it fits (K <= 8192), twice otherwise. Codes are
// round-to-nearest-even of the IEEE quotient x / scale, so they equal a plain fp32 statement of the same bit for bit.
//
// Reference counterparts: quant_rows_e4m3, absmax_cols_e4m3 / quant_cols_e4m3 (src/Idrak.Gpu/Cuda/PtxKernels.EightBit.cs:17-23).
#include "common.cuh"
#include <cuda_fp8.h>

namespace idrak {

constexpr float kE4m3Max = 448.f;

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return uint32_t(lo) | (uint32_t(hi) << 16);
}

// x: [rows, ld] bf16 (K valid columns, K % 8 == 0); q: [rows, ldq] bytes; scales: [rows]
template <int VPL>
__global__ void __launch_bounds__(256) quant_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ x, int ld,
                                                              uint8_t* __restrict__ q, int ldq,
                                                              float* __restrict__ scales, int rows, int K) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nvec = K >> 3;
  const __nv_bfloat16* xr = x + size_t(row) * ld;
  uint4 raw[VPL];
  float mx = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    raw[i] = (vi < nvec) ? *reinterpret_cast<const uint4*>(xr + vi * 8) : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w[k]);
      mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  mx = warp_max(mx);
  const float scale = mx > 0.f ? mx / kE4m3Max : 1.f;
  if (lane == 0) scales[row] = scale;
  uint8_t* qr = q + size_t(row) * ldq;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      const float2 a = unpack_bf16x2(raw[i].x), b = unpack_bf16x2(raw[i].y);
      const float2 c = unpack_bf16x2(raw[i].z), d = unpack_bf16x2(raw[i].w);
      uint2 o;
      o.x = pack_e4m3x4(a.x / scale, a.y / scale, b.x / scale, b.y / scale);
      o.y = pack_e4m3x4(c.x / scale, c.y / scale, d.x / scale, d.y / scale);
      *reinterpret_cast<uint2*>(qr + vi * 8) = o;
    }
  }
}

// Rows wider than the register budget: two passes over memory.
__global__ void __launch_bounds__(256) quant_rows_e4m3_stream_kernel(const __nv_bfloat16* __restrict__ x, int ld,
                                                                     uint8_t* __restrict__ q, int ldq,
                                                                     float* __restrict__ scales, int rows, int K) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nvec = K >> 3;
  const __nv_bfloat16* xr = x + size_t(row) * ld;
  float mx = 0.f;
  for (int vi = lane; vi < nvec; vi += 32) {
    const uint4 r = *reinterpret_cast<const uint4*>(xr + vi * 8);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w[k]);
      mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  mx = warp_max(mx);
  const float scale = mx > 0.f ? mx / kE4m3Max : 1.f;
  if (lane == 0) scales[row] = scale;
  uint8_t* qr = q + size_t(row) * ldq;
  for (int vi = lane; vi < nvec; vi += 32) {
    const uint4 r = *reinterpret_cast<const uint4*>(xr + vi * 8);
    const float2 a = unpack_bf16x2(r.x), b = unpack_bf16x2(r.y), c = unpack_bf16x2(r.z), d = unpack_bf16x2(r.w);
    uint2 o;
    o.x = pack_e4m3x4(a.x / scale, a.y / scale, b.x / scale, b.y / scale);
    o.y = pack_e4m3x4(c.x / scale, c.y / scale, d.x / scale, d.y / scale);
    *reinterpret_cast<uint2*>(qr + vi * 8) = o;
  }
}

// e4m3 codes back to bf16 (times the row scale): the check of a quantiser, and the fallback of a product whose
// sizes the 8-bit GEMM does not take.
__global__ void __launch_bounds__(256) dequant_rows_e4m3_kernel(const uint8_t* __restrict__ q, int ldq,
                                                                const float* __restrict__ scales,
                                                                __nv_bfloat16* __restrict__ x, int ld, int rows,
                                                                int K) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float s = scales[row];
  for (int c = lane * 2; c < K; c += 64) {
    const __nv_fp8x2_storage_t pair = *reinterpret_cast<const __nv_fp8x2_storage_t*>(q + size_t(row) * ldq + c);
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    *reinterpret_cast<uint32_t*>(x + size_t(row) * ld + c) = pack_bf16x2(f.x * s, f.y * s);
  }
}

}  // namespace idrak

using namespace idrak;

// x [rows, ld] bf16 -> q [rows, ldq] e4m3 codes + scales [rows]. K % 8 == 0, ld % 8 == 0, ldq % 8 == 0.
IDRAK_API int idrak_quant_rows_e4m3(const void* x, int ld, void* q, int ldq, float* scales, int rows, int K,
                                    void* stream_) {
  if (rows <= 0 || K <= 0) return 0;
  if ((K & 7) || (ld & 7) || (ldq & 7)) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  uint8_t* qp = static_cast<uint8_t*>(q);
  const int blocks = (rows + 7) / 8;
  const int nvec = K / 8;
  if (nvec <= 32 * 4) quant_rows_e4m3_kernel<4><<<blocks, 256, 0, s>>>(xp, ld, qp, ldq, scales, rows, K);
  else if (nvec <= 32 * 16) quant_rows_e4m3_kernel<16><<<blocks, 256, 0, s>>>(xp, ld, qp, ldq, scales, rows, K);
  else if (nvec <= 32 * 32) quant_rows_e4m3_kernel<32><<<blocks, 256, 0, s>>>(xp, ld, qp, ldq, scales, rows, K);
  else quant_rows_e4m3_stream_kernel<<<blocks, 256, 0, s>>>(xp, ld, qp, ldq, scales, rows, K);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_dequant_rows_e4m3(const void* q, int ldq, const float* scales, void* x, int ld, int rows, int K,
                                      void* stream_) {
  if (rows <= 0 || K <= 0) return 0;
  if ((K & 1) || (ld & 1) || (ldq & 1)) return -2;
  dequant_rows_e4m3_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(q), ldq, scales, static_cast<__nv_bfloat16*>(x), ld, rows, K);
  note_launches(1);
  return int(cudaGetLastError());
}
