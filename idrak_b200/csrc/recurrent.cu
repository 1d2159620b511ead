// LSTM and GRU cells: the element-wise half of a time step, forward and backward, fp32 or bf16 storage.
//
// A step of a recurrent layer is two products (input and hidden projections, run by the GEMM kernels: the input
// projection of a whole sequence is one many-row product, the hidden projection of a step a few-row one) followed by
// the gate arithmetic. That arithmetic is one launch here: it reads the pre-activation sums once, writes the new state
// and keeps the activated gates for the backward pass, which is again one launch per step producing the gradient of
// the pre-activation sums (what the weight-gradient products consume) and of the previous state.
//
// Gate order is (input, forget, cell, output) for the LSTM and (reset, update, new) for the GRU, the GRU's new-gate in
// the "reset after the product" form: n = tanh(gi_n + r * gh_n), h' = (1 - z) * n + z * h.
//
// Reference counterparts: lstm_cell / lstm_cell_bwd / gru_cell / gru_cell_bwd (src/Idrak.Gpu/Cuda/PtxKernels.Recurrent.cs).
#include "common.cuh"

namespace idrak {

template <class T> __device__ __forceinline__ float rld(const T* p);
template <> __device__ __forceinline__ float rld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float rld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <class T> __device__ __forceinline__ void rst(T* p, float v);
template <> __device__ __forceinline__ void rst<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void rst<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// gates [B, 4H] (sums of both projections and biases), c_prev [B, H] -> h, c [B, H]; acts [B, 4H] keeps the activated
// gates (i, f, g, o) for the backward pass.
template <class T>
__global__ void __launch_bounds__(256) lstm_cell_kernel(const T* __restrict__ gates, const T* __restrict__ c_prev,
                                                        T* __restrict__ h, T* __restrict__ c, T* __restrict__ acts,
                                                        int B, int H) {
  const long long n = (long long)B * H;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long b = idx / H;
    const int j = int(idx - b * H);
    const T* g = gates + b * 4 * H;
    const float i = sigmoid_f(rld(g + j));
    const float f = sigmoid_f(rld(g + H + j));
    const float gg = tanhf(rld(g + 2 * H + j));
    const float o = sigmoid_f(rld(g + 3 * H + j));
    const float cn = f * rld(c_prev + idx) + i * gg;
    rst(c + idx, cn);
    rst(h + idx, o * tanhf(cn));
    T* a = acts + b * 4 * H;
    rst(a + j, i);
    rst(a + H + j, f);
    rst(a + 2 * H + j, gg);
    rst(a + 3 * H + j, o);
  }
}

// dh, dc (gradients arriving at h and c of this step; dc may be null) -> dgates [B, 4H], dc_prev [B, H].
template <class T>
__global__ void __launch_bounds__(256) lstm_cell_bwd_kernel(const T* __restrict__ acts, const T* __restrict__ c_prev,
                                                            const T* __restrict__ c, const T* __restrict__ dh,
                                                            const T* __restrict__ dc, T* __restrict__ dgates,
                                                            T* __restrict__ dc_prev, int B, int H) {
  const long long n = (long long)B * H;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long b = idx / H;
    const int j = int(idx - b * H);
    const T* a = acts + b * 4 * H;
    const float i = rld(a + j), f = rld(a + H + j), gg = rld(a + 2 * H + j), o = rld(a + 3 * H + j);
    const float tc = tanhf(rld(c + idx));
    const float gh = rld(dh + idx);
    const float gc = (dc ? rld(dc + idx) : 0.f) + gh * o * (1.f - tc * tc);
    T* d = dgates + b * 4 * H;
    rst(d + j, gc * gg * i * (1.f - i));
    rst(d + H + j, gc * rld(c_prev + idx) * f * (1.f - f));
    rst(d + 2 * H + j, gc * i * (1.f - gg * gg));
    rst(d + 3 * H + j, gh * tc * o * (1.f - o));
    rst(dc_prev + idx, gc * f);
  }
}

// gi, gh [B, 3H] (input and hidden projections with their biases), h_prev [B, H] -> h [B, H];
// acts [B, 4H] keeps (r, z, n, gh_n) for the backward pass.
template <class T>
__global__ void __launch_bounds__(256) gru_cell_kernel(const T* __restrict__ gi, const T* __restrict__ gh,
                                                       const T* __restrict__ h_prev, T* __restrict__ h,
                                                       T* __restrict__ acts, int B, int H) {
  const long long n = (long long)B * H;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long b = idx / H;
    const int j = int(idx - b * H);
    const T* a = gi + b * 3 * H;
    const T* c = gh + b * 3 * H;
    const float r = sigmoid_f(rld(a + j) + rld(c + j));
    const float z = sigmoid_f(rld(a + H + j) + rld(c + H + j));
    const float hn = rld(c + 2 * H + j);
    const float nn = tanhf(rld(a + 2 * H + j) + r * hn);
    rst(h + idx, (1.f - z) * nn + z * rld(h_prev + idx));
    T* s = acts + b * 4 * H;
    rst(s + j, r);
    rst(s + H + j, z);
    rst(s + 2 * H + j, nn);
    rst(s + 3 * H + j, hn);
  }
}

// dh -> dgi, dgh [B, 3H] and dh_prev [B, H] (the part that does not pass through the hidden projection; the caller adds
// dgh * W_hh).
template <class T>
__global__ void __launch_bounds__(256) gru_cell_bwd_kernel(const T* __restrict__ acts, const T* __restrict__ h_prev,
                                                           const T* __restrict__ dh, T* __restrict__ dgi,
                                                           T* __restrict__ dgh, T* __restrict__ dh_prev, int B, int H) {
  const long long n = (long long)B * H;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long b = idx / H;
    const int j = int(idx - b * H);
    const T* s = acts + b * 4 * H;
    const float r = rld(s + j), z = rld(s + H + j), nn = rld(s + 2 * H + j), hn = rld(s + 3 * H + j);
    const float g = rld(dh + idx);
    const float dn = g * (1.f - z) * (1.f - nn * nn);
    const float dz = g * (rld(h_prev + idx) - nn) * z * (1.f - z);
    const float dr = dn * hn * r * (1.f - r);
    T* a = dgi + b * 3 * H;
    T* c = dgh + b * 3 * H;
    rst(a + j, dr);
    rst(a + H + j, dz);
    rst(a + 2 * H + j, dn);
    rst(c + j, dr);
    rst(c + H + j, dz);
    rst(c + 2 * H + j, dn * r);
    rst(dh_prev + idx, g * z);
  }
}

static inline int cell_grid(long long n) {
  const long long g = (n + 255) / 256, cap = (long long)sm_count() * 8;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace idrak

using namespace idrak;

#define RC_STREAM static_cast<cudaStream_t>(stream_)
#define RC_DISPATCH(dtype, ...)                                          \
  if (B < 1 || H < 1) return -2;                                         \
  if (dtype == 0) { using T = float; __VA_ARGS__; }                      \
  else if (dtype == 1) { using T = __nv_bfloat16; __VA_ARGS__; }         \
  else return -2;                                                        \
  note_launches(1);                                                      \
  return int(cudaGetLastError());
#define RC_C(p) static_cast<const T*>(p)
#define RC_M(p) static_cast<T*>(p)

IDRAK_API int idrak_lstm_cell(int dtype, const void* gates, const void* c_prev, void* h, void* c, void* acts, int B,
                              int H, void* stream_) {
  RC_DISPATCH(dtype, lstm_cell_kernel<T><<<cell_grid((long long)B * H), 256, 0, RC_STREAM>>>(
      RC_C(gates), RC_C(c_prev), RC_M(h), RC_M(c), RC_M(acts), B, H));
}
IDRAK_API int idrak_lstm_cell_bwd(int dtype, const void* acts, const void* c_prev, const void* c, const void* dh,
                                  const void* dc, void* dgates, void* dc_prev, int B, int H, void* stream_) {
  RC_DISPATCH(dtype, lstm_cell_bwd_kernel<T><<<cell_grid((long long)B * H), 256, 0, RC_STREAM>>>(
      RC_C(acts), RC_C(c_prev), RC_C(c), RC_C(dh), RC_C(dc), RC_M(dgates), RC_M(dc_prev), B, H));
}
IDRAK_API int idrak_gru_cell(int dtype, const void* gi, const void* gh, const void* h_prev, void* h, void* acts, int B,
                             int H, void* stream_) {
  RC_DISPATCH(dtype, gru_cell_kernel<T><<<cell_grid((long long)B * H), 256, 0, RC_STREAM>>>(
      RC_C(gi), RC_C(gh), RC_C(h_prev), RC_M(h), RC_M(acts), B, H));
}
IDRAK_API int idrak_gru_cell_bwd(int dtype, const void* acts, const void* h_prev, const void* dh, void* dgi, void* dgh,
                                 void* dh_prev, int B, int H, void* stream_) {
  RC_DISPATCH(dtype, gru_cell_bwd_kernel<T><<<cell_grid((long long)B * H), 256, 0, RC_STREAM>>>(
      RC_C(acts), RC_C(h_prev), RC_C(dh), RC_M(dgi), RC_M(dgh), RC_M(dh_prev), B, H));
}
