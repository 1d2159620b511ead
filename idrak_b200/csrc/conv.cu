// Convolution as patch matrices around the tensor-core GEMM, plus the kernels that have no product in them: depthwise
// convolution and max / average pooling, forward and backward. Tensors are N x C x H x W, fp32 or bf16.
//
// A dense convolution runs as   rows(N*OH*OW, C*KH*KW) x weight(OC, C*KH*KW)^T   on the tcgen05 GEMM:
//   im2col        unfolds the input into bf16 patch rows (row length padded to a multiple of 8 elements, the GEMM's
//                 16-byte rule for a leading dimension; the padding is written as zeros),
//   rows_to_nchw  turns the product's pixel-major result back into planes (and nchw_to_rows does the reverse for the
//                 incoming gradient),
//   col2im        folds the gradient of the patch rows back onto the input; each input pixel sums the patches that
//                 contain it, in a fixed order and without atomics.
// The weight gradient is the product rows(dy)^T x rows(x) on the same GEMM.
//
// Reference counterparts: im2col / col2im / maxpool (+bwd, +bwd_gather) (src/Idrak.Gpu/Cuda/PtxKernels.Advanced.cs:12),
// conv_fwd / conv_bwd_input / conv_bwd_weight / conv_dw (+bwd_input, +bwd_weight) / avgpool (+bwd)
// (PtxKernels.Convolution.cs).
#include "common.cuh"
#include <cfloat>

namespace idrak {

template <class T> __device__ __forceinline__ float cld(const T* p);
template <> __device__ __forceinline__ float cld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float cld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <class T> __device__ __forceinline__ void cst(T* p, float v);
template <> __device__ __forceinline__ void cst<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void cst<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

struct ConvShape {
  int N, C, H, W, KH, KW, OH, OW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
};

// rows[(n, oh, ow), (c, kh, kw)] = x[n, c, oh * s - p + kh * d, ow * s - p + kw * d] (0 outside); ld >= C * KH * KW.
template <class T>
__global__ void __launch_bounds__(256) im2col_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ rows,
                                                     ConvShape s, int ld) {
  const int K = s.C * s.KH * s.KW;
  const long long total = (long long)s.N * s.OH * s.OW * ld;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / ld;
    const int k = int(i - row * ld);
    float v = 0.f;
    if (k < K) {
      const int kw = k % s.KW, kh = (k / s.KW) % s.KH, c = k / (s.KW * s.KH);
      const int ow = int(row % s.OW), oh = int((row / s.OW) % s.OH);
      const long long n = row / ((long long)s.OW * s.OH);
      const int ih = oh * s.stride_h - s.pad_h + kh * s.dil_h, iw = ow * s.stride_w - s.pad_w + kw * s.dil_w;
      if (ih >= 0 && ih < s.H && iw >= 0 && iw < s.W) v = cld(x + ((n * s.C + c) * s.H + ih) * s.W + iw);
    }
    rows[i] = __float2bfloat16(v);
  }
}

// dx[n, c, ih, iw] = sum over the (kh, kw, oh, ow) whose patch element lands on that pixel of drows[...].
template <class T>
__global__ void __launch_bounds__(256) col2im_kernel(const __nv_bfloat16* __restrict__ drows, T* __restrict__ dx,
                                                     ConvShape s, int ld, int accumulate) {
  const long long total = (long long)s.N * s.C * s.H * s.W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int iw = int(i % s.W), ih = int((i / s.W) % s.H);
    const int c = int((i / ((long long)s.W * s.H)) % s.C);
    const long long n = i / ((long long)s.W * s.H * s.C);
    float acc = 0.f;
    for (int kh = 0; kh < s.KH; ++kh) {
      const int th = ih + s.pad_h - kh * s.dil_h;
      if (th < 0 || th % s.stride_h) continue;
      const int oh = th / s.stride_h;
      if (oh >= s.OH) continue;
      for (int kw = 0; kw < s.KW; ++kw) {
        const int tw = iw + s.pad_w - kw * s.dil_w;
        if (tw < 0 || tw % s.stride_w) continue;
        const int ow = tw / s.stride_w;
        if (ow >= s.OW) continue;
        const long long row = (n * s.OH + oh) * s.OW + ow;
        acc += __bfloat162float(drows[row * ld + (c * s.KH + kh) * s.KW + kw]);
      }
    }
    cst(dx + i, accumulate ? cld(dx + i) + acc : acc);
  }
}

// planes [N, C, P] <-> pixel rows [N * P, ld] (bf16), through a 32 x 33 tile so that both sides are coalesced.
template <class T>
__global__ void __launch_bounds__(256) nchw_to_rows_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ rows,
                                                           int C, int P, int ld) {
  __shared__ float tile[32][33];
  const T* xb = x + (long long)blockIdx.z * C * P;
  __nv_bfloat16* rb = rows + (long long)blockIdx.z * P * ld;
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8) {
    const int c = c0 + k, p = p0 + tx;
    tile[k][tx] = (c < C && p < P) ? cld(xb + (long long)c * P + p) : 0.f;
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int p = p0 + k, c = c0 + tx;
    if (p < P && c < ld) rb[(long long)p * ld + c] = __float2bfloat16(c < C ? tile[tx][k] : 0.f);
  }
}
// y[n, c, p] = rows[n * P + p, c] + (bias ? bias[c] : 0)
template <class T>
__global__ void __launch_bounds__(256) rows_to_nchw_kernel(const __nv_bfloat16* __restrict__ rows, T* __restrict__ y,
                                                           const float* __restrict__ bias, int C, int P, int ld) {
  __shared__ float tile[32][33];
  const __nv_bfloat16* rb = rows + (long long)blockIdx.z * P * ld;
  T* yb = y + (long long)blockIdx.z * C * P;
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8) {
    const int p = p0 + k, c = c0 + tx;
    tile[k][tx] = (p < P && c < C) ? __bfloat162float(rb[(long long)p * ld + c]) : 0.f;
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int c = c0 + k, p = p0 + tx;
    if (c < C && p < P) cst(yb + (long long)c * P + p, tile[tx][k] + (bias ? bias[c] : 0.f));
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// depthwise: weight [C, KH, KW] (multiplier 1)
template <class T>
__global__ void __launch_bounds__(256) dw_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                     const T* __restrict__ bias, T* __restrict__ y, ConvShape s) {
  const long long total = (long long)s.N * s.C * s.OH * s.OW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ow = int(i % s.OW), oh = int((i / s.OW) % s.OH);
    const long long plane = i / ((long long)s.OW * s.OH);
    const int c = int(plane % s.C);
    const T* xp = x + plane * s.H * s.W;
    const T* wp = w + (long long)c * s.KH * s.KW;
    float acc = bias ? cld(bias + c) : 0.f;
    for (int kh = 0; kh < s.KH; ++kh) {
      const int ih = oh * s.stride_h - s.pad_h + kh * s.dil_h;
      if (ih < 0 || ih >= s.H) continue;
      for (int kw = 0; kw < s.KW; ++kw) {
        const int iw = ow * s.stride_w - s.pad_w + kw * s.dil_w;
        if (iw < 0 || iw >= s.W) continue;
        acc += cld(xp + (long long)ih * s.W + iw) * cld(wp + kh * s.KW + kw);
      }
    }
    cst(y + i, acc);
  }
}
template <class T>
__global__ void __launch_bounds__(256) dw_bwd_input_kernel(const T* __restrict__ dy, const T* __restrict__ w,
                                                           T* __restrict__ dx, ConvShape s) {
  const long long total = (long long)s.N * s.C * s.H * s.W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int iw = int(i % s.W), ih = int((i / s.W) % s.H);
    const long long plane = i / ((long long)s.W * s.H);
    const int c = int(plane % s.C);
    const T* gp = dy + plane * s.OH * s.OW;
    const T* wp = w + (long long)c * s.KH * s.KW;
    float acc = 0.f;
    for (int kh = 0; kh < s.KH; ++kh) {
      const int th = ih + s.pad_h - kh * s.dil_h;
      if (th < 0 || th % s.stride_h) continue;
      const int oh = th / s.stride_h;
      if (oh >= s.OH) continue;
      for (int kw = 0; kw < s.KW; ++kw) {
        const int tw = iw + s.pad_w - kw * s.dil_w;
        if (tw < 0 || tw % s.stride_w) continue;
        const int ow = tw / s.stride_w;
        if (ow >= s.OW) continue;
        acc += cld(gp + (long long)oh * s.OW + ow) * cld(wp + kh * s.KW + kw);
      }
    }
    cst(dx + i, acc);
  }
}
// one block per (c, kh, kw): a fixed-order sum over images and output pixels. dbias (optional) by the kh = kw = 0 blocks.
template <class T>
__global__ void __launch_bounds__(256) dw_bwd_weight_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                            float* __restrict__ dw, float* __restrict__ dbias,
                                                            ConvShape s) {
  __shared__ float part[2][8];
  const int kw = blockIdx.x % s.KW, kh = (blockIdx.x / s.KW) % s.KH, c = blockIdx.x / (s.KW * s.KH);
  const long long per = (long long)s.OH * s.OW, total = (long long)s.N * per;
  float acc = 0.f, bsum = 0.f;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    const long long n = i / per;
    const int ow = int(i % s.OW), oh = int((i / s.OW) % s.OH);
    const float g = cld(dy + ((n * s.C + c) * s.OH + oh) * s.OW + ow);
    bsum += g;
    const int ih = oh * s.stride_h - s.pad_h + kh * s.dil_h, iw = ow * s.stride_w - s.pad_w + kw * s.dil_w;
    if (ih >= 0 && ih < s.H && iw >= 0 && iw < s.W) acc += g * cld(x + ((n * s.C + c) * s.H + ih) * s.W + iw);
  }
  acc = warp_sum(acc);
  bsum = warp_sum(bsum);
  if ((threadIdx.x & 31) == 0) { part[0][threadIdx.x >> 5] = acc; part[1][threadIdx.x >> 5] = bsum; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int w = 0; w < 8; ++w) { a += part[0][w]; b += part[1][w]; }
    dw[blockIdx.x] = a;
    if (dbias && kh == 0 && kw == 0) dbias[c] = b;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// pooling over planes [N * C, H, W]. Max pooling keeps the flat index (ih * W + iw) of the winner, first on a tie.
template <class T>
__global__ void __launch_bounds__(256) maxpool_kernel(const T* __restrict__ x, T* __restrict__ y, int* __restrict__ index,
                                                      ConvShape s) {
  const long long total = (long long)s.N * s.C * s.OH * s.OW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ow = int(i % s.OW), oh = int((i / s.OW) % s.OH);
    const long long plane = i / ((long long)s.OW * s.OH);
    const T* xp = x + plane * s.H * s.W;
    float best = -FLT_MAX;
    int bi = -1;
    for (int kh = 0; kh < s.KH; ++kh) {
      const int ih = oh * s.stride_h - s.pad_h + kh * s.dil_h;
      if (ih < 0 || ih >= s.H) continue;
      for (int kw = 0; kw < s.KW; ++kw) {
        const int iw = ow * s.stride_w - s.pad_w + kw * s.dil_w;
        if (iw < 0 || iw >= s.W) continue;
        const float v = cld(xp + (long long)ih * s.W + iw);
        if (v > best || bi < 0) { best = v; bi = ih * s.W + iw; }
      }
    }
    cst(y + i, best);
    if (index) index[i] = bi;
  }
}
// gather form: an input pixel collects dy from the windows that chose it
template <class T>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const T* __restrict__ dy, const int* __restrict__ index,
                                                          T* __restrict__ dx, ConvShape s) {
  const long long total = (long long)s.N * s.C * s.H * s.W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int iw = int(i % s.W), ih = int((i / s.W) % s.H);
    const long long plane = i / ((long long)s.W * s.H);
    const int me = ih * s.W + iw;
    float acc = 0.f;
    for (int kh = 0; kh < s.KH; ++kh) {
      const int th = ih + s.pad_h - kh * s.dil_h;
      if (th < 0 || th % s.stride_h) continue;
      const int oh = th / s.stride_h;
      if (oh >= s.OH) continue;
      for (int kw = 0; kw < s.KW; ++kw) {
        const int tw = iw + s.pad_w - kw * s.dil_w;
        if (tw < 0 || tw % s.stride_w) continue;
        const int ow = tw / s.stride_w;
        if (ow >= s.OW) continue;
        const long long o = (plane * s.OH + oh) * s.OW + ow;
        if (index[o] == me) acc += cld(dy + o);
      }
    }
    cst(dx + i, acc);
  }
}
// average pooling; include_pad: divide by the window size, else by the number of pixels inside the image
template <class T>
__global__ void __launch_bounds__(256) avgpool_kernel(const T* __restrict__ x, T* __restrict__ y, ConvShape s,
                                                      int include_pad) {
  const long long total = (long long)s.N * s.C * s.OH * s.OW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ow = int(i % s.OW), oh = int((i / s.OW) % s.OH);
    const long long plane = i / ((long long)s.OW * s.OH);
    const T* xp = x + plane * s.H * s.W;
    float acc = 0.f;
    int inside = 0;
    for (int kh = 0; kh < s.KH; ++kh) {
      const int ih = oh * s.stride_h - s.pad_h + kh;
      if (ih < 0 || ih >= s.H) continue;
      for (int kw = 0; kw < s.KW; ++kw) {
        const int iw = ow * s.stride_w - s.pad_w + kw;
        if (iw < 0 || iw >= s.W) continue;
        acc += cld(xp + (long long)ih * s.W + iw);
        ++inside;
      }
    }
    const int div = include_pad ? s.KH * s.KW : max(inside, 1);
    cst(y + i, acc / float(div));
  }
}
template <class T>
__global__ void __launch_bounds__(256) avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, ConvShape s,
                                                          int include_pad) {
  const long long total = (long long)s.N * s.C * s.H * s.W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int iw = int(i % s.W), ih = int((i / s.W) % s.H);
    const long long plane = i / ((long long)s.W * s.H);
    float acc = 0.f;
    for (int kh = 0; kh < s.KH; ++kh) {
      const int th = ih + s.pad_h - kh;
      if (th < 0 || th % s.stride_h) continue;
      const int oh = th / s.stride_h;
      if (oh >= s.OH) continue;
      for (int kw = 0; kw < s.KW; ++kw) {
        const int tw = iw + s.pad_w - kw;
        if (tw < 0 || tw % s.stride_w) continue;
        const int ow = tw / s.stride_w;
        if (ow >= s.OW) continue;
        int div = s.KH * s.KW;
        if (!include_pad) {
          const int h0 = max(oh * s.stride_h - s.pad_h, 0), h1 = min(oh * s.stride_h - s.pad_h + s.KH, s.H);
          const int w0 = max(ow * s.stride_w - s.pad_w, 0), w1 = min(ow * s.stride_w - s.pad_w + s.KW, s.W);
          div = max((h1 - h0) * (w1 - w0), 1);
        }
        acc += cld(dy + (plane * s.OH + oh) * s.OW + ow) / float(div);
      }
    }
    cst(dx + i, acc);
  }
}

static inline int conv_grid(long long n) {
  const long long g = (n + 255) / 256, cap = (long long)sm_count() * 8;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}
static inline bool shape_ok(const ConvShape& s) {
  return s.N > 0 && s.C > 0 && s.H > 0 && s.W > 0 && s.KH > 0 && s.KW > 0 && s.OH > 0 && s.OW > 0 && s.stride_h > 0 &&
         s.stride_w > 0 && s.dil_h > 0 && s.dil_w > 0 && s.pad_h >= 0 && s.pad_w >= 0;
}

}  // namespace idrak

using namespace idrak;

#define CV_STREAM static_cast<cudaStream_t>(stream_)
#define CV_DISPATCH(dtype, ...)                                          \
  if (dtype == 0) { using T = float; __VA_ARGS__; }                      \
  else if (dtype == 1) { using T = __nv_bfloat16; __VA_ARGS__; }         \
  else return -2;                                                        \
  note_launches(1);                                                      \
  return int(cudaGetLastError());
#define CV_C(p) static_cast<const T*>(p)
#define CV_M(p) static_cast<T*>(p)

// `shape`: the 14 integers of ConvShape in declaration order.
static inline ConvShape shape_from(const int* v) {
  ConvShape s{v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11], v[12], v[13]};
  return s;
}

IDRAK_API int idrak_im2col(int dtype, const void* x, void* rows, const int* shape, int ld, void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s) || ld < s.C * s.KH * s.KW) return -2;
  CV_DISPATCH(dtype, im2col_kernel<T><<<conv_grid((long long)s.N * s.OH * s.OW * ld), 256, 0, CV_STREAM>>>(
      CV_C(x), static_cast<__nv_bfloat16*>(rows), s, ld));
}
IDRAK_API int idrak_col2im(int dtype, const void* drows, void* dx, const int* shape, int ld, int accumulate,
                           void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s) || ld < s.C * s.KH * s.KW) return -2;
  CV_DISPATCH(dtype, col2im_kernel<T><<<conv_grid((long long)s.N * s.C * s.H * s.W), 256, 0, CV_STREAM>>>(
      static_cast<const __nv_bfloat16*>(drows), CV_M(dx), s, ld, accumulate));
}
IDRAK_API int idrak_nchw_to_rows(int dtype, const void* x, void* rows, int N, int C, int P, int ld, void* stream_) {
  if (N < 1 || N > 65535 || C < 1 || P < 1 || ld < C || (ld + 31) / 32 > 65535) return -2;
  const dim3 grid((P + 31) / 32, (ld + 31) / 32, N);
  CV_DISPATCH(dtype, nchw_to_rows_kernel<T><<<grid, 256, 0, CV_STREAM>>>(CV_C(x), static_cast<__nv_bfloat16*>(rows), C,
                                                                        P, ld));
}
IDRAK_API int idrak_rows_to_nchw(int dtype, const void* rows, void* y, const float* bias, int N, int C, int P, int ld,
                                 void* stream_) {
  if (N < 1 || N > 65535 || C < 1 || P < 1 || ld < C || (C + 31) / 32 > 65535) return -2;
  const dim3 grid((P + 31) / 32, (C + 31) / 32, N);
  CV_DISPATCH(dtype, rows_to_nchw_kernel<T><<<grid, 256, 0, CV_STREAM>>>(static_cast<const __nv_bfloat16*>(rows),
                                                                        CV_M(y), bias, C, P, ld));
}
IDRAK_API int idrak_dw_conv(int dtype, const void* x, const void* w, const void* bias, void* y, const int* shape,
                            void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s)) return -2;
  CV_DISPATCH(dtype, dw_fwd_kernel<T><<<conv_grid((long long)s.N * s.C * s.OH * s.OW), 256, 0, CV_STREAM>>>(
      CV_C(x), CV_C(w), CV_C(bias), CV_M(y), s));
}
IDRAK_API int idrak_dw_conv_bwd_input(int dtype, const void* dy, const void* w, void* dx, const int* shape,
                                      void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s)) return -2;
  CV_DISPATCH(dtype, dw_bwd_input_kernel<T><<<conv_grid((long long)s.N * s.C * s.H * s.W), 256, 0, CV_STREAM>>>(
      CV_C(dy), CV_C(w), CV_M(dx), s));
}
// dw [C, KH, KW] and dbias [C] (optional) in fp32
IDRAK_API int idrak_dw_conv_bwd_weight(int dtype, const void* x, const void* dy, float* dw, float* dbias,
                                       const int* shape, void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s)) return -2;
  CV_DISPATCH(dtype, dw_bwd_weight_kernel<T><<<s.C * s.KH * s.KW, 256, 0, CV_STREAM>>>(CV_C(x), CV_C(dy), dw, dbias, s));
}
IDRAK_API int idrak_maxpool(int dtype, const void* x, void* y, int* index, const int* shape, void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s)) return -2;
  CV_DISPATCH(dtype, maxpool_kernel<T><<<conv_grid((long long)s.N * s.C * s.OH * s.OW), 256, 0, CV_STREAM>>>(
      CV_C(x), CV_M(y), index, s));
}
IDRAK_API int idrak_maxpool_bwd(int dtype, const void* dy, const int* index, void* dx, const int* shape,
                                void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s)) return -2;
  CV_DISPATCH(dtype, maxpool_bwd_kernel<T><<<conv_grid((long long)s.N * s.C * s.H * s.W), 256, 0, CV_STREAM>>>(
      CV_C(dy), index, CV_M(dx), s));
}
IDRAK_API int idrak_avgpool(int dtype, const void* x, void* y, const int* shape, int include_pad, void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s)) return -2;
  CV_DISPATCH(dtype, avgpool_kernel<T><<<conv_grid((long long)s.N * s.C * s.OH * s.OW), 256, 0, CV_STREAM>>>(
      CV_C(x), CV_M(y), s, include_pad));
}
IDRAK_API int idrak_avgpool_bwd(int dtype, const void* dy, void* dx, const int* shape, int include_pad, void* stream_) {
  const ConvShape s = shape_from(shape);
  if (!shape_ok(s)) return -2;
  CV_DISPATCH(dtype, avgpool_bwd_kernel<T><<<conv_grid((long long)s.N * s.C * s.H * s.W), 256, 0, CV_STREAM>>>(
      CV_C(dy), CV_M(dx), s, include_pad));
}
