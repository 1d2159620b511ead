// AdamW with 8-bit moments: m and v live as one byte per value, scaled per block of 256 values by that block's
// largest magnitude. A byte indexes a fixed non-linear map (denser near zero): signed for m, unsigned for v.
// One CTA per block of 256 values: de-quantise both moments, apply the update in fp32, find the new block maxima
// with a CTA reduction, re-quantise, write the parameter (fp32 master and, when given, its bf16 shadow).
// Optimizer state costs 2 bytes per parameter (+ 8 bytes per 256) instead of 8.
//
// Reference: adam8_f32 and EightBitMoments (src/Idrak.Gpu/Cuda/PtxKernels.Rows.cs:258,
// src/Idrak.Abstraction/Devices/Backend.cs:2099).
#include "common.cuh"

namespace idrak {

constexpr int kAdam8Block = 256;

// code <-> value in [-1, 1] (signed) or [0, 1] (unsigned); the map is x |x| on a uniform grid, so it is monotone
// and its inverse is a square root.
__device__ __forceinline__ float adam8_signed_value(uint8_t c) {
  const float x = (float(c) - 127.5f) * (1.f / 127.5f);
  return x * fabsf(x);
}
__device__ __forceinline__ uint8_t adam8_signed_code(float y) {
  const float x = copysignf(sqrtf(fabsf(y)), y);
  return uint8_t(min(255, max(0, __float2int_rn(x * 127.5f + 127.5f))));
}
__device__ __forceinline__ float adam8_unsigned_value(uint8_t c) {
  const float x = float(c) * (1.f / 255.f);
  return x * x;
}
__device__ __forceinline__ uint8_t adam8_unsigned_code(float y) {
  // round up: a small second moment must not collapse to zero (it is a denominator)
  const float x = sqrtf(fmaxf(y, 0.f)) * 255.f;
  return uint8_t(min(255, max(y > 0.f ? 1 : 0, int(ceilf(x - 1e-4f)))));
}

struct Adam8Hyper {
  float lr, beta1, beta2, eps, bc1, bc2, weight_decay, grad_scale;
};

__global__ void __launch_bounds__(kAdam8Block) adam8_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow,
                                                            const void* __restrict__ grad, int grad_bf16,
                                                            uint8_t* __restrict__ m8, uint8_t* __restrict__ v8,
                                                            float* __restrict__ m_absmax, float* __restrict__ v_absmax,
                                                            long long n, Adam8Hyper h, const float* __restrict__ clip) {
  __shared__ float red_m[kAdam8Block / 32], red_v[kAdam8Block / 32];
  const long long i = (long long)blockIdx.x * kAdam8Block + threadIdx.x;
  const bool live = i < n;
  const float scale = h.grad_scale * (clip ? *clip : 1.f);
  float p = 0.f, m = 0.f, v = 0.f;
  if (live) {
    const float g = (grad_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(grad)[i])
                               : static_cast<const float*>(grad)[i]) * scale;
    p = master[i];
    m = adam8_signed_value(m8[i]) * m_absmax[blockIdx.x];
    v = adam8_unsigned_value(v8[i]) * v_absmax[blockIdx.x];
    m = h.beta1 * m + (1.f - h.beta1) * g;
    v = h.beta2 * v + (1.f - h.beta2) * g * g;
    const float update = (m / h.bc1) / (sqrtf(v / h.bc2) + h.eps);
    p = p * (1.f - h.lr * h.weight_decay) - h.lr * update;
  }
  float am = warp_max(fabsf(m)), av = warp_max(v);
  if ((threadIdx.x & 31) == 0) { red_m[threadIdx.x >> 5] = am; red_v[threadIdx.x >> 5] = av; }
  __syncthreads();
  am = red_m[0]; av = red_v[0];
#pragma unroll
  for (int w = 1; w < kAdam8Block / 32; ++w) { am = fmaxf(am, red_m[w]); av = fmaxf(av, red_v[w]); }
  if (live) {
    master[i] = p;
    if (shadow) shadow[i] = __float2bfloat16(p);
    m8[i] = adam8_signed_code(am > 0.f ? m / am : 0.f);
    v8[i] = adam8_unsigned_code(av > 0.f ? v / av : 0.f);
  }
  if (threadIdx.x == 0) { m_absmax[blockIdx.x] = am; v_absmax[blockIdx.x] = av; }
}

}  // namespace idrak

using namespace idrak;

IDRAK_API int idrak_adam8_block() { return kAdam8Block; }

// One parameter tensor of n values. m8 / v8: n bytes each (zero-initialised = zero moments for the signed map's
// code 128 / unsigned code 0: callers fill m8 with 128); m_absmax / v_absmax: ceil(n / 256) floats.
IDRAK_API int idrak_adam8_step(float* master, void* shadow_bf16, const void* grad, int grad_bf16, void* m8, void* v8,
                               float* m_absmax, float* v_absmax, long long n, float lr, float beta1, float beta2,
                               float eps, float bc1, float bc2, float weight_decay, float grad_scale,
                               const float* clip_factor, void* stream_) {
  if (n <= 0) return 0;
  Adam8Hyper h{lr, beta1, beta2, eps, bc1, bc2, weight_decay, grad_scale};
  const long long blocks = (n + kAdam8Block - 1) / kAdam8Block;
  if (blocks > 0x7fffffffLL) return -2;
  adam8_kernel<<<int(blocks), kAdam8Block, 0, static_cast<cudaStream_t>(stream_)>>>(
      master, static_cast<__nv_bfloat16*>(shadow_bf16), grad, grad_bf16, static_cast<uint8_t*>(m8),
      static_cast<uint8_t*>(v8), m_absmax, v_absmax, n, h, clip_factor);
  note_launches(1);
  return int(cudaGetLastError());
}
