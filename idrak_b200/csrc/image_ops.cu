// Image-side kernels: fused resize + normalise of decoded images (uint8 HWC -> float / bf16 CHW), nearest / bilinear
// interpolation and adaptive average / max pooling on NCHW tensors, each with its backward pass.
// All are bandwidth-bound gather / scatter kernels: one thread per output element, coalesced along the output
// row; backward passes of interpolation and average pooling gather from the output gradient (no atomics), so the
// results do not depend on scheduling.
//
// Reference: ResizeNormalize and the resampling family interpolate(+bwd), adaptive_{avg,max}pool(+bwd)
// (src/Idrak.Gpu/Cuda/PtxKernels.Resampling.cs; host contract src/Idrak.Abstraction/Tensors/Tensor.Resampling.cs).
#include "common.cuh"

namespace idrak {

template <typename T> __device__ __forceinline__ float ld_f(const T* p, size_t i);
template <> __device__ __forceinline__ float ld_f<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __bfloat162float(p[i]);
}
template <typename T> __device__ __forceinline__ void st_f(T* p, size_t i, float v);
template <> __device__ __forceinline__ void st_f<float>(float* p, size_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, size_t i, float v) {
  p[i] = __float2bfloat16(v);
}

// source coordinate of output index o under "half-pixel centres" (align_corners = false)
__device__ __forceinline__ float src_coord(int o, float scale) { return fmaxf((o + 0.5f) * scale - 0.5f, 0.f); }

// ---------------------------------------------------------------------------------------------------------------
// uint8 [N, H, W, C] -> T [N, C, OH, OW]: bilinear resize, then (v / 255 - mean[c]) / std[c]
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) resize_normalize_kernel(const uint8_t* __restrict__ src, T* __restrict__ dst, int N,
                                                               int H, int W, int C, int OH, int OW,
                                                               const float* __restrict__ mean,
                                                               const float* __restrict__ inv_std, int nearest) {
  const long long total = (long long)N * C * OH * OW;
  const float sy = float(H) / OH, sx = float(W) / OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ox = int(i % OW);
    const int oy = int((i / OW) % OH);
    const int c = int((i / ((long long)OW * OH)) % C);
    const int n = int(i / ((long long)OW * OH * C));
    const uint8_t* img = src + size_t(n) * H * W * C;
    float v;
    if (nearest) {
      const int y = min(int(floorf(oy * sy)), H - 1), x = min(int(floorf(ox * sx)), W - 1);
      v = img[(size_t(y) * W + x) * C + c];
    } else {
      const float fy = src_coord(oy, sy), fx = src_coord(ox, sx);
      const int y0 = min(int(fy), H - 1), x0 = min(int(fx), W - 1);
      const int y1 = min(y0 + 1, H - 1), x1 = min(x0 + 1, W - 1);
      const float wy = fy - y0, wx = fx - x0;
      const float a = img[(size_t(y0) * W + x0) * C + c], b = img[(size_t(y0) * W + x1) * C + c];
      const float d = img[(size_t(y1) * W + x0) * C + c], e = img[(size_t(y1) * W + x1) * C + c];
      v = (a * (1.f - wx) + b * wx) * (1.f - wy) + (d * (1.f - wx) + e * wx) * wy;
    }
    st_f(dst, size_t(i), (v * (1.f / 255.f) - mean[c]) * inv_std[c]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// interpolate on [planes = N * C, H, W] -> [planes, OH, OW]
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) interpolate_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long planes,
                                                              int H, int W, int OH, int OW, int bilinear) {
  const long long total = planes * OH * OW;
  const float sy = float(H) / OH, sx = float(W) / OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ox = int(i % OW), oy = int((i / OW) % OH);
    const long long p = i / ((long long)OW * OH);
    const T* img = x + size_t(p) * H * W;
    float v;
    if (!bilinear) {
      const int yy = min(int(floorf(oy * sy)), H - 1), xx = min(int(floorf(ox * sx)), W - 1);
      v = ld_f(img, size_t(yy) * W + xx);
    } else {
      const float fy = src_coord(oy, sy), fx = src_coord(ox, sx);
      const int y0 = min(int(fy), H - 1), x0 = min(int(fx), W - 1);
      const int y1 = min(y0 + 1, H - 1), x1 = min(x0 + 1, W - 1);
      const float wy = fy - y0, wx = fx - x0;
      v = (ld_f(img, size_t(y0) * W + x0) * (1.f - wx) + ld_f(img, size_t(y0) * W + x1) * wx) * (1.f - wy) +
          (ld_f(img, size_t(y1) * W + x0) * (1.f - wx) + ld_f(img, size_t(y1) * W + x1) * wx) * wy;
    }
    st_f(y, size_t(i), v);
  }
}

// dx[p, h, w] = sum over the output pixels that read (h, w) of their weight * dy. Gathered per input pixel over the
// bounded range of output pixels that can touch it, in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256) interpolate_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, long long planes,
                                                              int H, int W, int OH, int OW, int bilinear) {
  const long long total = planes * H * W;
  const float sy = float(H) / OH, sx = float(W) / OW;
  const float ry = float(OH) / H, rx = float(OW) / W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int w = int(i % W), h = int((i / W) % H);
    const long long p = i / ((long long)W * H);
    const T* g = dy + size_t(p) * OH * OW;
    // output rows / columns whose source coordinate can fall in [h - 1, h + 1]
    const int oy_lo = max(0, int(floorf((h - 1) * ry)) - 1), oy_hi = min(OH - 1, int(ceilf((h + 2) * ry)) + 1);
    const int ox_lo = max(0, int(floorf((w - 1) * rx)) - 1), ox_hi = min(OW - 1, int(ceilf((w + 2) * rx)) + 1);
    float acc = 0.f;
    for (int oy = oy_lo; oy <= oy_hi; ++oy) {
      float wy;
      if (!bilinear) {
        wy = (min(int(floorf(oy * sy)), H - 1) == h) ? 1.f : 0.f;
      } else {
        const float fy = src_coord(oy, sy);
        const int y0 = min(int(fy), H - 1), y1 = min(y0 + 1, H - 1);
        const float t = fy - y0;
        wy = (y0 == h ? 1.f - t : 0.f) + (y1 == h ? t : 0.f);
      }
      if (wy == 0.f) continue;
      for (int ox = ox_lo; ox <= ox_hi; ++ox) {
        float wx;
        if (!bilinear) {
          wx = (min(int(floorf(ox * sx)), W - 1) == w) ? 1.f : 0.f;
        } else {
          const float fx = src_coord(ox, sx);
          const int x0 = min(int(fx), W - 1), x1 = min(x0 + 1, W - 1);
          const float t = fx - x0;
          wx = (x0 == w ? 1.f - t : 0.f) + (x1 == w ? t : 0.f);
        }
        if (wx != 0.f) acc += wy * wx * ld_f(g, size_t(oy) * OW + ox);
      }
    }
    st_f(dx, size_t(i), acc);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// adaptive pooling on [planes, H, W] -> [planes, OH, OW]; window of output o: [floor(o H / OH), ceil((o + 1) H / OH))
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ int win_lo(int o, int in, int out) { return int((long long)o * in / out); }
__device__ __forceinline__ int win_hi(int o, int in, int out) { return int(((long long)(o + 1) * in + out - 1) / out); }

template <typename T>
__global__ void __launch_bounds__(256) adaptive_pool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                int* __restrict__ index, long long planes, int H, int W,
                                                                int OH, int OW, int is_max) {
  const long long total = planes * OH * OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ox = int(i % OW), oy = int((i / OW) % OH);
    const long long p = i / ((long long)OW * OH);
    const T* img = x + size_t(p) * H * W;
    const int y0 = win_lo(oy, H, OH), y1 = win_hi(oy, H, OH), x0 = win_lo(ox, W, OW), x1 = win_hi(ox, W, OW);
    if (is_max) {
      float best = -INFINITY;
      int where = y0 * W + x0;
      for (int yy = y0; yy < y1; ++yy)
        for (int xx = x0; xx < x1; ++xx) {
          const float v = ld_f(img, size_t(yy) * W + xx);
          if (v > best || v != v) { best = v; where = yy * W + xx; }     // first maximum; NaN propagates
        }
      st_f(y, size_t(i), best);
      if (index) index[i] = where;
    } else {
      float s = 0.f;
      for (int yy = y0; yy < y1; ++yy)
        for (int xx = x0; xx < x1; ++xx) s += ld_f(img, size_t(yy) * W + xx);
      st_f(y, size_t(i), s / float((y1 - y0) * (x1 - x0)));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) adaptive_pool_bwd_kernel(const T* __restrict__ dy, const int* __restrict__ index,
                                                                T* __restrict__ dx, long long planes, int H, int W, int OH,
                                                                int OW, int is_max) {
  const long long total = planes * H * W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int w = int(i % W), h = int((i / W) % H);
    const long long p = i / ((long long)W * H);
    const T* g = dy + size_t(p) * OH * OW;
    // outputs whose window holds (h, w)
    int oy_lo = int((long long)h * OH / H), ox_lo = int((long long)w * OW / W);
    while (oy_lo > 0 && win_hi(oy_lo - 1, H, OH) > h) --oy_lo;
    while (ox_lo > 0 && win_hi(ox_lo - 1, W, OW) > w) --ox_lo;
    float acc = 0.f;
    for (int oy = oy_lo; oy < OH && win_lo(oy, H, OH) <= h; ++oy) {
      if (win_hi(oy, H, OH) <= h) continue;
      for (int ox = ox_lo; ox < OW && win_lo(ox, W, OW) <= w; ++ox) {
        if (win_hi(ox, W, OW) <= w) continue;
        const size_t o = size_t(oy) * OW + ox;
        if (is_max) {
          if (index[size_t(p) * OH * OW + o] == h * W + w) acc += ld_f(g, o);
        } else {
          const int area = (win_hi(oy, H, OH) - win_lo(oy, H, OH)) * (win_hi(ox, W, OW) - win_lo(ox, W, OW));
          acc += ld_f(g, o) / float(area);
        }
      }
    }
    st_f(dx, size_t(i), acc);
  }
}

static int blocks_for(long long n) {
  long long b = (n + 255) / 256, cap = (long long)sm_count() * 16;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace idrak

using namespace idrak;

#define IDRAK_BY_TYPE(bf16, CALL_F32, CALL_BF16) \
  do { if (bf16) { CALL_BF16; } else { CALL_F32; } } while (0)

IDRAK_API int idrak_resize_normalize(const void* src, void* dst, int bf16, int N, int H, int W, int C, int OH, int OW,
                                     const float* mean, const float* inv_std, int nearest, void* stream_) {
  if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || OH <= 0 || OW <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int grid = blocks_for((long long)N * C * OH * OW);
  IDRAK_BY_TYPE(bf16,
      (resize_normalize_kernel<float><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(src), static_cast<float*>(dst), N, H,
                                                           W, C, OH, OW, mean, inv_std, nearest)),
      (resize_normalize_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(src),
                                                                   static_cast<__nv_bfloat16*>(dst), N, H, W, C, OH, OW,
                                                                   mean, inv_std, nearest)));
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_interpolate(const void* x, void* y, int bf16, long long planes, int H, int W, int OH, int OW,
                                int bilinear, int backward, void* stream_) {
  if (planes <= 0 || H <= 0 || W <= 0 || OH <= 0 || OW <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  if (!backward) {
    const int grid = blocks_for(planes * OH * OW);
    IDRAK_BY_TYPE(bf16,
        (interpolate_fwd_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(y), planes, H,
                                                            W, OH, OW, bilinear)),
        (interpolate_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                                    static_cast<__nv_bfloat16*>(y), planes, H, W, OH, OW,
                                                                    bilinear)));
  } else {   // x = dy [planes, OH, OW], y = dx [planes, H, W]
    const int grid = blocks_for(planes * H * W);
    IDRAK_BY_TYPE(bf16,
        (interpolate_bwd_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(y), planes, H,
                                                            W, OH, OW, bilinear)),
        (interpolate_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                                    static_cast<__nv_bfloat16*>(y), planes, H, W, OH, OW,
                                                                    bilinear)));
  }
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_adaptive_pool(const void* x, void* y, int* index, int bf16, long long planes, int H, int W, int OH,
                                  int OW, int is_max, int backward, void* stream_) {
  if (planes <= 0 || H <= 0 || W <= 0 || OH <= 0 || OW <= 0) return -2;
  if (backward && is_max && index == nullptr) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  if (!backward) {
    const int grid = blocks_for(planes * OH * OW);
    IDRAK_BY_TYPE(bf16,
        (adaptive_pool_fwd_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(y), index,
                                                              planes, H, W, OH, OW, is_max)),
        (adaptive_pool_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                                      static_cast<__nv_bfloat16*>(y), index, planes, H, W,
                                                                      OH, OW, is_max)));
  } else {   // x = dy, y = dx
    const int grid = blocks_for(planes * H * W);
    IDRAK_BY_TYPE(bf16,
        (adaptive_pool_bwd_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), index, static_cast<float*>(y),
                                                              planes, H, W, OH, OW, is_max)),
        (adaptive_pool_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), index,
                                                                      static_cast<__nv_bfloat16*>(y), planes, H, W, OH,
                                                                      OW, is_max)));
  }
  note_launches(1);
  return int(cudaGetLastError());
}
