// Row reductions and index kernels over fp32 or bf16 storage: softmax and log-softmax (forward, backward, and the
// scaled / masked form attention scores take when they are materialised), sums along an axis and its inverse
// (broadcast), permutation of up to six axes with a tiled path for a swap of the two innermost ones, row gather,
// one-hot, and the count of rows whose arg-max equals a target.
//
// Reductions run in a fixed order (lane-strided partial sums, then a shuffle butterfly, then a fixed walk over the
// warps' partials), never through floating-point atomics, so a rerun gives the same bits.
//
// Reference counterparts: softmax_f32 / softmax_bwd / argmax / class_match / gather_f32 / one_hot / permute / sum_axis /
// sum_axis_rows / broadcast_axis (src/Idrak.Gpu/Cuda/PtxKernels.Advanced.cs:12), transpose_f32 / sum_rows_f32
// (PtxKernels.Rows.cs:231-660), scale_mask_softmax_f32 (PtxKernels.Decoding.cs:12).
#include "common.cuh"
#include <cfloat>

namespace idrak {

template <class T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <class T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

constexpr int kRowThreads = 256;

// Block-wide reductions of (value) with a fixed order: warp butterflies, then thread 0..7 partials summed by every thread
// in the same order.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float s = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) s += scratch[w];
  return s;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float s = -FLT_MAX;
  for (int w = 0; w < (blockDim.x >> 5); ++w) s = fmaxf(s, scratch[w]);
  return s;
}

// ---------------------------------------------------------------------------------------------------------------------
// softmax over the last axis. One block per row (rows in a grid-stride loop). The score of column c of row r is
//   s = scale * x[r, c] + (mask ? mask[(r % mask_rows), c] : 0),  minus infinity where causal and c > (r % tq) + shift.
// `log_form` writes s - max - log(sum) instead of the probability. A row with every column masked gives zeros.
template <class T>
__global__ void __launch_bounds__(kRowThreads) softmax_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                              long long rows, int cols, float scale,
                                                              const float* __restrict__ mask, int mask_rows, int causal,
                                                              int tq, int shift, int log_form) {
  __shared__ float scratch[kRowThreads / 32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    T* yr = y + r * cols;
    const int limit = causal ? min(cols, int(r % tq) + shift + 1) : cols;
    const float* mr = mask ? mask + (long long)(r % mask_rows) * cols : nullptr;
    float m = -FLT_MAX;
    for (int c = threadIdx.x; c < limit; c += blockDim.x) {
      const float s = scale * ldf(xr + c) + (mr ? mr[c] : 0.f);
      m = fmaxf(m, s);
    }
    m = block_max(m, scratch);
    float sum = 0.f;
    for (int c = threadIdx.x; c < limit; c += blockDim.x) {
      const float s = scale * ldf(xr + c) + (mr ? mr[c] : 0.f);
      sum += __expf(s - m);
    }
    sum = block_sum(sum, scratch);
    const bool empty = !(sum > 0.f) || m == -FLT_MAX;
    const float inv = empty ? 0.f : 1.f / sum;
    const float lse = empty ? 0.f : m + __logf(sum);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float out;
      if (c < limit && !empty) {
        const float s = scale * ldf(xr + c) + (mr ? mr[c] : 0.f);
        out = log_form ? s - lse : __expf(s - m) * inv;
      } else {
        out = log_form ? -FLT_MAX : 0.f;
      }
      stf(yr + c, out);
    }
  }
}

// softmax:      dx = scale * y * (dy - sum(dy * y))
// log-softmax:  dx = scale * (dy - exp(y) * sum(dy))
template <class T>
__global__ void __launch_bounds__(kRowThreads) softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy,
                                                                  T* __restrict__ dx, long long rows, int cols,
                                                                  float scale, int log_form) {
  __shared__ float scratch[kRowThreads / 32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* yr = y + r * cols;
    const T* gr = dy + r * cols;
    T* dr = dx + r * cols;
    float dot = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float yv = ldf(yr + c), g = ldf(gr + c);
      if (log_form) dot += (yv > -FLT_MAX * 0.5f) ? g : 0.f;
      else dot += g * yv;
    }
    dot = block_sum(dot, scratch);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float yv = ldf(yr + c), g = ldf(gr + c);
      float out;
      if (log_form) out = (yv > -FLT_MAX * 0.5f) ? g - __expf(yv) * dot : 0.f;
      else out = yv * (g - dot);
      stf(dr + c, scale * out);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// x viewed as [outer, axis, inner] -> out[outer, inner] (fp32). inner == 1: one block per row. Otherwise one thread per
// output element walks the axis (neighbouring threads read neighbouring addresses).
template <class T>
__global__ void __launch_bounds__(kRowThreads) sum_rows_kernel(const T* __restrict__ x, float* __restrict__ out,
                                                               long long rows, long long cols, float scale) {
  __shared__ float scratch[kRowThreads / 32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * cols;
    float s = 0.f;
    for (long long c = threadIdx.x; c < cols; c += blockDim.x) s += ldf(xr + c);
    s = block_sum(s, scratch);
    if (threadIdx.x == 0) out[r] = s * scale;
  }
}
template <class T>
__global__ void __launch_bounds__(256) sum_axis_kernel(const T* __restrict__ x, float* __restrict__ out, long long outer,
                                                       int axis, long long inner, float scale) {
  const long long total = outer * inner;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long o = i / inner, in = i - o * inner;
    const T* p = x + o * axis * inner + in;
    float s = 0.f;
    for (int a = 0; a < axis; ++a) s += ldf(p + a * inner);
    out[i] = s * scale;
  }
}
// The same sum when there are few outputs and a long axis: one block per (32 inner positions, outer index), eight warps
// stride the axis and their partial sums are added in warp order.
template <class T>
__global__ void __launch_bounds__(256) sum_axis_tiled_kernel(const T* __restrict__ x, float* __restrict__ out, int axis,
                                                             long long inner, float scale) {
  __shared__ float part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long in = (long long)blockIdx.x * 32 + tx;
  const long long o = blockIdx.y;
  float s = 0.f;
  if (in < inner) {
    const T* p = x + o * axis * inner + in;
    for (int a = ty; a < axis; a += 8) s += ldf(p + a * inner);
  }
  part[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && in < inner) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += part[w][tx];
    out[o * inner + in] = t * scale;
  }
}
// out[o, a, i] = (accumulate ? out : 0) + x[o, i]
template <class T>
__global__ void __launch_bounds__(256) broadcast_axis_kernel(const float* __restrict__ x, T* __restrict__ out,
                                                             long long outer, int axis, long long inner,
                                                             int accumulate) {
  const long long total = outer * axis * inner;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long in = i % inner, o = i / (inner * axis);
    const float v = x[o * inner + in];
    stf(out + i, accumulate ? ldf(out + i) + v : v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
struct PermuteDims {
  int rank;
  long long out_dim[6];      // extents of the result, outermost first
  long long src_stride[6];   // stride (in elements) in the source of each result axis
};
template <class T>
__global__ void __launch_bounds__(256) permute_kernel(const T* __restrict__ x, T* __restrict__ y, long long n,
                                                      PermuteDims d) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    long long rest = i, src = 0;
#pragma unroll
    for (int k = 5; k >= 0; --k) {
      if (k < d.rank) {
        const long long q = rest / d.out_dim[k];
        src += (rest - q * d.out_dim[k]) * d.src_stride[k];
        rest = q;
      }
    }
    y[i] = x[src];
  }
}
// y[b, c, r] = x[b, r, c] through a 32 x 33 shared tile: both sides coalesced.
template <class T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols) {
  __shared__ T tile[32][33];
  const long long plane = (long long)rows * cols;
  const T* xb = x + blockIdx.z * plane;
  T* yb = y + blockIdx.z * plane;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8) {
    const int r = r0 + k, c = c0 + tx;
    if (r < rows && c < cols) tile[k][tx] = xb[(long long)r * cols + c];
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int c = c0 + k, r = r0 + tx;
    if (r < rows && c < cols) yb[(long long)c * rows + r] = tile[tx][k];
  }
}

// out[r, :] = table[ids[r], :]; an id outside the table gives a row of zeros.
template <class T>
__global__ void __launch_bounds__(256) gather_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                                          T* __restrict__ out, long long rows, int cols,
                                                          long long table_rows) {
  const long long total = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = int(i - r * cols);
    const long long id = ids[r];
    out[i] = (id >= 0 && id < table_rows) ? table[id * cols + c] : T(0.f);
  }
}
template <class T>
__global__ void __launch_bounds__(256) one_hot_kernel(const int* __restrict__ ids, T* __restrict__ out, long long rows,
                                                      int classes) {
  const long long total = rows * classes;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / classes;
    stf(out + i, int(i - r * classes) == ids[r] ? 1.f : 0.f);
  }
}

// Adds to *count the number of rows whose arg-max (lowest index on a tie) equals targets[r]; rows with a negative target
// are left out. Integer atomics: the total does not depend on the order.
template <class T>
__global__ void __launch_bounds__(kRowThreads) class_match_kernel(const T* __restrict__ logits,
                                                                  const int* __restrict__ targets, long long rows,
                                                                  int cols, int* __restrict__ count) {
  __shared__ float best_v[kRowThreads / 32];
  __shared__ int best_i[kRowThreads / 32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const int target = targets[r];
    if (target < 0) continue;
    const T* xr = logits + r * cols;
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float v = ldf(xr + c);
      if (v > bv) { bv = v; bi = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < kRowThreads / 32; ++w)
        if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
      if (bi == target) atomicAdd(count, 1);
    }
  }
}

static inline int rows_grid(long long rows) {
  const long long cap = (long long)sm_count() * 8;
  return int(rows < 1 ? 1 : (rows > cap ? cap : rows));
}
static inline int flat_grid(long long n) {
  const long long g = (n + 255) / 256, cap = (long long)sm_count() * 8;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace idrak

using namespace idrak;

#define RD_STREAM static_cast<cudaStream_t>(stream_)
#define RD_DISPATCH(dtype, ...)                                          \
  if (dtype == 0) { using T = float; __VA_ARGS__; }                      \
  else if (dtype == 1) { using T = __nv_bfloat16; __VA_ARGS__; }         \
  else return -2;                                                        \
  note_launches(1);                                                      \
  return int(cudaGetLastError());

// mask: optional fp32 [mask_rows, cols] added to the scaled scores (row r uses mask row r % mask_rows).
// causal: column c of row r is kept when c <= (r % tq) + shift.
IDRAK_API int idrak_softmax(int dtype, const void* x, void* y, long long rows, int cols, float scale, const float* mask,
                            int mask_rows, int causal, int tq, int shift, int log_form, void* stream_) {
  if (cols < 1 || (mask && mask_rows < 1) || (causal && tq < 1)) return -2;
  RD_DISPATCH(dtype, softmax_kernel<T><<<rows_grid(rows), kRowThreads, 0, RD_STREAM>>>(
      static_cast<const T*>(x), static_cast<T*>(y), rows, cols, scale, mask, mask ? mask_rows : 1, causal,
      causal ? tq : 1, shift, log_form));
}
IDRAK_API int idrak_softmax_bwd(int dtype, const void* y, const void* dy, void* dx, long long rows, int cols,
                                float scale, int log_form, void* stream_) {
  if (cols < 1) return -2;
  RD_DISPATCH(dtype, softmax_bwd_kernel<T><<<rows_grid(rows), kRowThreads, 0, RD_STREAM>>>(
      static_cast<const T*>(y), static_cast<const T*>(dy), static_cast<T*>(dx), rows, cols, scale, log_form));
}
IDRAK_API int idrak_sum_axis(int dtype, const void* x, float* out, long long outer, int axis, long long inner,
                             float scale, void* stream_) {
  if (outer < 1 || axis < 1 || inner < 1) return -2;
  if (inner == 1) {
    RD_DISPATCH(dtype, sum_rows_kernel<T><<<rows_grid(outer), kRowThreads, 0, RD_STREAM>>>(
        static_cast<const T*>(x), out, outer, axis, scale));
  }
  if (outer * inner < 65536 && axis >= 64 && outer <= 65535) {
    const dim3 grid((unsigned)((inner + 31) / 32), (unsigned)outer);
    RD_DISPATCH(dtype, sum_axis_tiled_kernel<T><<<grid, 256, 0, RD_STREAM>>>(static_cast<const T*>(x), out, axis, inner,
                                                                            scale));
  }
  RD_DISPATCH(dtype, sum_axis_kernel<T><<<flat_grid(outer * inner), 256, 0, RD_STREAM>>>(
      static_cast<const T*>(x), out, outer, axis, inner, scale));
}
IDRAK_API int idrak_broadcast_axis(int dtype, const float* x, void* out, long long outer, int axis, long long inner,
                                   int accumulate, void* stream_) {
  if (outer < 1 || axis < 1 || inner < 1) return -2;
  RD_DISPATCH(dtype, broadcast_axis_kernel<T><<<flat_grid(outer * axis * inner), 256, 0, RD_STREAM>>>(
      x, static_cast<T*>(out), outer, axis, inner, accumulate));
}
// out_dims: extents of the result; src_strides: the source stride (elements) of each result axis; rank <= 6.
IDRAK_API int idrak_permute(int dtype, const void* x, void* y, int rank, const long long* out_dims,
                            const long long* src_strides, void* stream_) {
  if (rank < 1 || rank > 6) return -2;
  PermuteDims d{};
  d.rank = rank;
  long long n = 1;
  for (int k = 0; k < rank; ++k) {
    d.out_dim[k] = out_dims[k];
    d.src_stride[k] = src_strides[k];
    n *= out_dims[k];
  }
  if (n < 1) return -2;
  RD_DISPATCH(dtype, permute_kernel<T><<<flat_grid(n), 256, 0, RD_STREAM>>>(static_cast<const T*>(x),
                                                                          static_cast<T*>(y), n, d));
}
IDRAK_API int idrak_transpose(int dtype, const void* x, void* y, int batch, int rows, int cols, void* stream_) {
  if (batch < 1 || batch > 65535 || rows < 1 || cols < 1 || (rows + 31) / 32 > 65535) return -2;
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
  RD_DISPATCH(dtype, transpose_kernel<T><<<grid, 256, 0, RD_STREAM>>>(static_cast<const T*>(x), static_cast<T*>(y),
                                                                     rows, cols));
}
IDRAK_API int idrak_gather_rows(int dtype, const void* table, const int* ids, void* out, long long rows, int cols,
                                long long table_rows, void* stream_) {
  if (rows < 1 || cols < 1) return -2;
  RD_DISPATCH(dtype, gather_rows_kernel<T><<<flat_grid(rows * cols), 256, 0, RD_STREAM>>>(
      static_cast<const T*>(table), ids, static_cast<T*>(out), rows, cols, table_rows));
}
IDRAK_API int idrak_one_hot(int dtype, const int* ids, void* out, long long rows, int classes, void* stream_) {
  if (rows < 1 || classes < 1) return -2;
  RD_DISPATCH(dtype, one_hot_kernel<T><<<flat_grid(rows * classes), 256, 0, RD_STREAM>>>(ids, static_cast<T*>(out),
                                                                                       rows, classes));
}
// *count must be zeroed by the caller (or hold a running total).
IDRAK_API int idrak_class_match(int dtype, const void* logits, const int* targets, long long rows, int cols, int* count,
                                void* stream_) {
  if (rows < 1 || cols < 1) return -2;
  RD_DISPATCH(dtype, class_match_kernel<T><<<rows_grid(rows), kRowThreads, 0, RD_STREAM>>>(
      static_cast<const T*>(logits), targets, rows, cols, count));
}
