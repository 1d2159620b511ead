// Element-wise kernels over contiguous tensors, fp32 or bf16 storage with fp32 arithmetic.
//
// One kernel per arity, not one per function: the operation is a code the whole grid agrees on, so the switch costs a
// few uniform instructions next to a 128-bit load and store per eight (bf16) or four (fp32) elements. The kernels are
// bandwidth-bound; a grid-stride loop over vectors keeps the grid at a few CTAs per SM, and a scalar tail takes what is
// left when the element count is not a multiple of the vector width. Backward kernels recompute the function from the
// saved input (or take the saved output where the derivative is cheaper from it) and either write or accumulate.
//
// Dropout keeps no mask: element i of a call draws from a counter-based generator keyed by (seed, i), so the backward
// pass (and a rerun) sees the same draw.
//
// Reference counterparts: fill / affine / axpy / muladd / add / sub / mul / sigmoid / tanh / relu / square / abs (+_bwd),
// dropout, add_dropout, add_rowvec, add_scalar (src/Idrak.Gpu/Cuda/PtxKernels.cs:31-39), sqrt / sin / cos / silu / sign /
// max / min / extremum_bwd / pow / clamp / leaky_relu / where (PtxKernels.Pointwise.cs), exp / log / gelu / gelu_erf /
// inv_sqrt (PtxKernels.Advanced.cs:12).
#include "common.cuh"

namespace idrak {

enum UnaryOp : int {
  U_AFFINE = 0, U_SIGMOID, U_TANH, U_RELU, U_SQUARE, U_ABS, U_SQRT, U_SIN, U_COS, U_SILU, U_SIGN, U_EXP, U_LOG,
  U_GELU, U_GELU_ERF, U_INV_SQRT, U_POW, U_CLAMP, U_LEAKY_RELU, U_NEG, U_RECIPROCAL, U_COUNT
};
enum BinaryOp : int { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_MAX, B_MIN, B_AXPBY, B_COUNT };

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float gelu_tanh_d(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}

__device__ __forceinline__ float unary_f(int op, float x, float a, float b) {
  switch (op) {
    case U_AFFINE: return fmaf(a, x, b);
    case U_SIGMOID: return 1.f / (1.f + __expf(-x));
    case U_TANH: return tanhf(x);
    case U_RELU: return fmaxf(x, 0.f);
    case U_SQUARE: return x * x;
    case U_ABS: return fabsf(x);
    case U_SQRT: return sqrtf(x);
    case U_SIN: return sinf(x);
    case U_COS: return cosf(x);
    case U_SILU: return x / (1.f + __expf(-x));
    case U_SIGN: return float(x > 0.f) - float(x < 0.f);
    case U_EXP: return expf(x);
    case U_LOG: return logf(x);
    case U_GELU: return gelu_tanh_f(x);
    case U_GELU_ERF: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    case U_INV_SQRT: return rsqrtf(x + a);
    case U_POW: return powf(x, a);
    case U_CLAMP: return fminf(fmaxf(x, a), b);
    case U_LEAKY_RELU: return x > 0.f ? x : a * x;
    case U_NEG: return -x;
    case U_RECIPROCAL: return 1.f / x;
  }
  return x;
}

// d f(x) / dx, from the input
__device__ __forceinline__ float unary_d(int op, float x, float a, float b) {
  switch (op) {
    case U_AFFINE: return a;
    case U_SIGMOID: { const float s = 1.f / (1.f + __expf(-x)); return s * (1.f - s); }
    case U_TANH: { const float t = tanhf(x); return 1.f - t * t; }
    case U_RELU: return x > 0.f ? 1.f : 0.f;
    case U_SQUARE: return 2.f * x;
    case U_ABS: return float(x > 0.f) - float(x < 0.f);
    case U_SQRT: return 0.5f * rsqrtf(x);
    case U_SIN: return cosf(x);
    case U_COS: return -sinf(x);
    case U_SILU: { const float s = 1.f / (1.f + __expf(-x)); return s * (1.f + x * (1.f - s)); }
    case U_SIGN: return 0.f;
    case U_EXP: return expf(x);
    case U_LOG: return 1.f / x;
    case U_GELU: return gelu_tanh_d(x);
    case U_GELU_ERF:
      return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
    case U_INV_SQRT: { const float r = rsqrtf(x + a); return -0.5f * r * r * r; }
    case U_POW: return a * powf(x, a - 1.f);
    case U_CLAMP: return (x >= a && x <= b) ? 1.f : 0.f;
    case U_LEAKY_RELU: return x > 0.f ? 1.f : a;
    case U_NEG: return -1.f;
    case U_RECIPROCAL: return -1.f / (x * x);
  }
  return 1.f;
}

__device__ __forceinline__ float binary_f(int op, float x, float y, float a, float b) {
  switch (op) {
    case B_ADD: return x + y;
    case B_SUB: return x - y;
    case B_MUL: return x * y;
    case B_DIV: return x / y;
    case B_MAX: return fmaxf(x, y);
    case B_MIN: return fminf(x, y);
    case B_AXPBY: return fmaf(a, x, b * y);
  }
  return x;
}

// ---------------------------------------------------------------------------------------------------------------------
// vectors: V elements of T in one 16-byte access, as floats
template <class T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  __device__ static float get(const float* p) { return *p; }
  __device__ static void put(float* p, float v) { *p = v; }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    float2 f;
    f = unpack_bf16x2(a.x); v[0] = f.x; v[1] = f.y;
    f = unpack_bf16x2(a.y); v[2] = f.x; v[3] = f.y;
    f = unpack_bf16x2(a.z); v[4] = f.x; v[5] = f.y;
    f = unpack_bf16x2(a.w); v[6] = f.x; v[7] = f.y;
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = o;
  }
  __device__ static float get(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void put(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};

// Runs `f(i, vector?)` over n elements: whole vectors in a grid-stride loop, then the scalar tail.
template <class T, class FV, class FS>
__device__ __forceinline__ void for_each(long long n, FV fv, FS fs) {
  constexpr int N = Vec<T>::N;
  const long long nvec = n / N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) fv(i * N);
  const long long tail = nvec * N;
  for (long long i = tail + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) fs(i);
}

template <class T>
__global__ void __launch_bounds__(256) unary_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, int op,
                                                    float a, float b) {
  constexpr int N = Vec<T>::N;
  for_each<T>(n,
      [&](long long i) {
        float v[N];
        Vec<T>::load(x + i, v);
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = unary_f(op, v[j], a, b);
        Vec<T>::store(y + i, v);
      },
      [&](long long i) { Vec<T>::put(y + i, unary_f(op, Vec<T>::get(x + i), a, b)); });
}

// dx = (accumulate ? dx : 0) + dy * f'(x)
template <class T>
__global__ void __launch_bounds__(256) unary_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                        T* __restrict__ dx, long long n, int op, float a, float b,
                                                        int accumulate) {
  constexpr int N = Vec<T>::N;
  for_each<T>(n,
      [&](long long i) {
        float v[N], g[N], o[N];
        Vec<T>::load(x + i, v);
        Vec<T>::load(dy + i, g);
        if (accumulate) Vec<T>::load(dx + i, o);
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = (accumulate ? o[j] : 0.f) + g[j] * unary_d(op, v[j], a, b);
        Vec<T>::store(dx + i, o);
      },
      [&](long long i) {
        const float o = accumulate ? Vec<T>::get(dx + i) : 0.f;
        Vec<T>::put(dx + i, o + Vec<T>::get(dy + i) * unary_d(op, Vec<T>::get(x + i), a, b));
      });
}

template <class T>
__global__ void __launch_bounds__(256) binary_kernel(const T* __restrict__ x, const T* __restrict__ y,
                                                     T* __restrict__ out, long long n, int op, float a, float b) {
  constexpr int N = Vec<T>::N;
  for_each<T>(n,
      [&](long long i) {
        float u[N], v[N];
        Vec<T>::load(x + i, u);
        Vec<T>::load(y + i, v);
#pragma unroll
        for (int j = 0; j < N; ++j) u[j] = binary_f(op, u[j], v[j], a, b);
        Vec<T>::store(out + i, u);
      },
      [&](long long i) { Vec<T>::put(out + i, binary_f(op, Vec<T>::get(x + i), Vec<T>::get(y + i), a, b)); });
}

// out = x * y + z
template <class T>
__global__ void __launch_bounds__(256) muladd_kernel(const T* __restrict__ x, const T* __restrict__ y,
                                                     const T* __restrict__ z, T* __restrict__ out, long long n) {
  constexpr int N = Vec<T>::N;
  for_each<T>(n,
      [&](long long i) {
        float u[N], v[N], w[N];
        Vec<T>::load(x + i, u);
        Vec<T>::load(y + i, v);
        Vec<T>::load(z + i, w);
#pragma unroll
        for (int j = 0; j < N; ++j) u[j] = fmaf(u[j], v[j], w[j]);
        Vec<T>::store(out + i, u);
      },
      [&](long long i) {
        Vec<T>::put(out + i, fmaf(Vec<T>::get(x + i), Vec<T>::get(y + i), Vec<T>::get(z + i)));
      });
}

// Gradient of max / min: the whole of dy goes to the operand that was taken (the first on a tie).
template <class T>
__global__ void __launch_bounds__(256) extremum_bwd_kernel(const T* __restrict__ x, const T* __restrict__ y,
                                                           const T* __restrict__ dy, T* __restrict__ dx,
                                                           T* __restrict__ dyo, long long n, int is_max) {
  constexpr int N = Vec<T>::N;
  for_each<T>(n,
      [&](long long i) {
        float u[N], v[N], g[N], gx[N], gy[N];
        Vec<T>::load(x + i, u);
        Vec<T>::load(y + i, v);
        Vec<T>::load(dy + i, g);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const bool first = is_max ? (u[j] >= v[j]) : (u[j] <= v[j]);
          gx[j] = first ? g[j] : 0.f;
          gy[j] = first ? 0.f : g[j];
        }
        Vec<T>::store(dx + i, gx);
        Vec<T>::store(dyo + i, gy);
      },
      [&](long long i) {
        const float u = Vec<T>::get(x + i), v = Vec<T>::get(y + i), g = Vec<T>::get(dy + i);
        const bool first = is_max ? (u >= v) : (u <= v);
        Vec<T>::put(dx + i, first ? g : 0.f);
        Vec<T>::put(dyo + i, first ? 0.f : g);
      });
}

// out = cond ? x : y   (cond: one byte per element, non-zero = true)
template <class T>
__global__ void __launch_bounds__(256) where_kernel(const uint8_t* __restrict__ cond, const T* __restrict__ x,
                                                    const T* __restrict__ y, T* __restrict__ out, long long n) {
  constexpr int N = Vec<T>::N;
  for_each<T>(n,
      [&](long long i) {
        float u[N], v[N];
        Vec<T>::load(x + i, u);
        Vec<T>::load(y + i, v);
#pragma unroll
        for (int j = 0; j < N; ++j) u[j] = cond[i + j] ? u[j] : v[j];
        Vec<T>::store(out + i, u);
      },
      [&](long long i) { Vec<T>::put(out + i, cond[i] ? Vec<T>::get(x + i) : Vec<T>::get(y + i)); });
}

template <class T>
__global__ void __launch_bounds__(256) fill_kernel(T* __restrict__ out, long long n, float value) {
  constexpr int N = Vec<T>::N;
  for_each<T>(n,
      [&](long long i) {
        float v[N];
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = value;
        Vec<T>::store(out + i, v);
      },
      [&](long long i) { Vec<T>::put(out + i, value); });
}

// out[r, c] = x[r, c] + v[c]; cols a multiple of the vector width
template <class T>
__global__ void __launch_bounds__(256) add_rowvec_kernel(const T* __restrict__ x, const T* __restrict__ vec,
                                                         T* __restrict__ out, long long n, int cols) {
  constexpr int N = Vec<T>::N;
  for_each<T>(n,
      [&](long long i) {
        float u[N], v[N];
        Vec<T>::load(x + i, u);
        Vec<T>::load(vec + (i % cols), v);
#pragma unroll
        for (int j = 0; j < N; ++j) u[j] += v[j];
        Vec<T>::store(out + i, u);
      },
      [&](long long i) { Vec<T>::put(out + i, Vec<T>::get(x + i) + Vec<T>::get(vec + (i % cols))); });
}

// Counter-based uniform draw in [0, 1): two rounds of a 64-bit mix of (seed, index).
__device__ __forceinline__ float uniform_at(unsigned long long seed, unsigned long long i) {
  unsigned long long z = seed + (i + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return float(unsigned(z >> 40)) * (1.f / 16777216.f);
}

// out = (residual ? residual : 0) + keep(i) * x / (1 - p). The same kernel is the backward pass (x = dy, no residual).
template <class T>
__global__ void __launch_bounds__(256) dropout_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                                                      T* __restrict__ out, long long n, float p,
                                                      unsigned long long seed) {
  constexpr int N = Vec<T>::N;
  const float scale = 1.f / (1.f - p);
  for_each<T>(n,
      [&](long long i) {
        float u[N], r[N];
        Vec<T>::load(x + i, u);
        if (residual) Vec<T>::load(residual + i, r);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float kept = uniform_at(seed, (unsigned long long)(i + j)) >= p ? u[j] * scale : 0.f;
          u[j] = residual ? r[j] + kept : kept;
        }
        Vec<T>::store(out + i, u);
      },
      [&](long long i) {
        const float kept = uniform_at(seed, (unsigned long long)i) >= p ? Vec<T>::get(x + i) * scale : 0.f;
        Vec<T>::put(out + i, residual ? Vec<T>::get(residual + i) + kept : kept);
      });
}

static inline int pw_grid(long long n, int per_thread) {
  long long work = (n + per_thread - 1) / per_thread;
  long long g = (work + 255) / 256;
  long long cap = (long long)sm_count() * 8;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace idrak

using namespace idrak;

#define PW_STREAM static_cast<cudaStream_t>(stream_)
#define PW_DISPATCH(dtype, ...)                                          \
  if (dtype == 0) { using T = float; __VA_ARGS__; }                             \
  else if (dtype == 1) { using T = __nv_bfloat16; __VA_ARGS__; }               \
  else return -2;                                                        \
  note_launches(1);                                                      \
  return int(cudaGetLastError());

// dtype: 0 = fp32, 1 = bf16. Every pointer must be 16-byte aligned (returns -3 otherwise).
IDRAK_API int idrak_pw_unary(int op, int dtype, const void* x, void* y, long long n, float a, float b, void* stream_) {
  if (op < 0 || op >= U_COUNT) return -2;
  if (!aligned16(x) || !aligned16(y)) return -3;
  PW_DISPATCH(dtype, unary_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(
      static_cast<const T*>(x), static_cast<T*>(y), n, op, a, b));
}
IDRAK_API int idrak_pw_unary_bwd(int op, int dtype, const void* x, const void* dy, void* dx, long long n, float a,
                                 float b, int accumulate, void* stream_) {
  if (op < 0 || op >= U_COUNT) return -2;
  if (!aligned16(x) || !aligned16(dy) || !aligned16(dx)) return -3;
  PW_DISPATCH(dtype, unary_bwd_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(
      static_cast<const T*>(x), static_cast<const T*>(dy), static_cast<T*>(dx), n, op, a, b, accumulate));
}
IDRAK_API int idrak_pw_binary(int op, int dtype, const void* x, const void* y, void* out, long long n, float a,
                              float b, void* stream_) {
  if (op < 0 || op >= B_COUNT) return -2;
  if (!aligned16(x) || !aligned16(y) || !aligned16(out)) return -3;
  PW_DISPATCH(dtype, binary_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(
      static_cast<const T*>(x), static_cast<const T*>(y), static_cast<T*>(out), n, op, a, b));
}
IDRAK_API int idrak_pw_muladd(int dtype, const void* x, const void* y, const void* z, void* out, long long n,
                              void* stream_) {
  if (!aligned16(x) || !aligned16(y) || !aligned16(z) || !aligned16(out)) return -3;
  PW_DISPATCH(dtype, muladd_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(
      static_cast<const T*>(x), static_cast<const T*>(y), static_cast<const T*>(z), static_cast<T*>(out), n));
}
IDRAK_API int idrak_pw_extremum_bwd(int dtype, const void* x, const void* y, const void* dy, void* dx, void* dyo,
                                    long long n, int is_max, void* stream_) {
  if (!aligned16(x) || !aligned16(y) || !aligned16(dy) || !aligned16(dx) || !aligned16(dyo)) return -3;
  PW_DISPATCH(dtype, extremum_bwd_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(
      static_cast<const T*>(x), static_cast<const T*>(y), static_cast<const T*>(dy), static_cast<T*>(dx),
      static_cast<T*>(dyo), n, is_max));
}
IDRAK_API int idrak_pw_where(int dtype, const void* cond, const void* x, const void* y, void* out, long long n,
                             void* stream_) {
  if (!aligned16(x) || !aligned16(y) || !aligned16(out)) return -3;
  PW_DISPATCH(dtype, where_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(
      static_cast<const uint8_t*>(cond), static_cast<const T*>(x), static_cast<const T*>(y), static_cast<T*>(out), n));
}
IDRAK_API int idrak_pw_fill(int dtype, void* out, long long n, float value, void* stream_) {
  if (!aligned16(out)) return -3;
  PW_DISPATCH(dtype, fill_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(static_cast<T*>(out), n, value));
}
IDRAK_API int idrak_pw_add_rowvec(int dtype, const void* x, const void* vec, void* out, long long rows, int cols,
                                  void* stream_) {
  if (!aligned16(x) || !aligned16(vec) || !aligned16(out)) return -3;
  if (cols % (dtype == 0 ? 4 : 8)) return -2;
  const long long n = rows * cols;
  PW_DISPATCH(dtype, add_rowvec_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(
      static_cast<const T*>(x), static_cast<const T*>(vec), static_cast<T*>(out), n, cols));
}
// residual may be null. Backward: call it again with x = dy, residual = null and the same seed.
IDRAK_API int idrak_pw_dropout(int dtype, const void* x, const void* residual, void* out, long long n, float p,
                               unsigned long long seed, void* stream_) {
  if (!(p >= 0.f && p < 1.f)) return -2;
  if (!aligned16(x) || !aligned16(out) || (residual && !aligned16(residual))) return -3;
  PW_DISPATCH(dtype, dropout_kernel<T><<<pw_grid(n, Vec<T>::N), 256, 0, PW_STREAM>>>(
      static_cast<const T*>(x), static_cast<const T*>(residual), static_cast<T*>(out), n, p, seed));
}
