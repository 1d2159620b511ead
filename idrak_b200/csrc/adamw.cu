// Fused multi-tensor AdamW with global-norm clipping, and SGD with momentum.
//
// One launch covers every parameter: block b takes chunk b of a chunk table whose entries name a tensor
// and a first element. Three passes, none of which returns to the host:
//   1. multi_sumsq   per-chunk sums of squared gradients            -> partial[chunks]
//   2. clip_factor   ordered sum of the partials, norm, clip scale  -> hyper block on the device
//   3. multi_adamw   moments, decoupled decay, update of the fp32 master weight and of its bf16 copy;
//                    optionally zeroes the gradient so the next backward pass can accumulate into it
// Hyper-parameters (lr, betas, bias corrections ...) live in a small device block so a CUDA graph that
// recorded the launches keeps working as they change from step to step.
//
// Reference counterparts: multi_sumsq_f32 / sum_blocks_f32 / clip_factor_f32 / multi_adamw_f32 with the
// 40-byte tensor table and 4,096-element chunks (src/Idrak.Gpu/Cuda/PtxKernels.Rows.cs:508-598),
// Adam.ClipAndStep (src/Idrak.Abstraction/Training/Adam.cs:80-112), sgd_momentum_f32.
#include "common.cuh"

namespace idrak {

constexpr int kOptChunk = 4096;
constexpr int kOptThreads = 256;

struct OptTensor {        // one per parameter, in device memory
  float* master;          // fp32 weights (always)
  __nv_bfloat16* shadow;  // bf16 copy the model computes with (may be null)
  void* grad;             // bf16 or fp32
  float* m;
  float* v;
  long long n;
  float weight_decay;
  int grad_fp32;
};

struct OptChunk {
  int tensor;
  int pad;
  long long first;
};

// hyper block layout (floats)
enum { kHLr = 0, kHBeta1, kHBeta2, kHEps, kHBc1, kHBc2, kHClipScale, kHGradNorm, kHMaxNorm, kHGradScale, kHCount };

__device__ __forceinline__ float load_grad(const OptTensor& t, long long i) {
  return t.grad_fp32 ? static_cast<const float*>(t.grad)[i]
                     : __bfloat162float(static_cast<const __nv_bfloat16*>(t.grad)[i]);
}

__global__ void __launch_bounds__(kOptThreads) multi_sumsq_kernel(const OptTensor* __restrict__ tensors,
                                                                  const OptChunk* __restrict__ chunks,
                                                                  float* __restrict__ partial) {
  __shared__ float sm[kOptThreads / 32];
  const OptChunk c = chunks[blockIdx.x];
  const OptTensor t = tensors[c.tensor];
  const long long end = min(t.n, c.first + kOptChunk);
  float s = 0.f;
  for (long long i = c.first + threadIdx.x; i < end; i += kOptThreads) {
    float g = load_grad(t, i);
    s += g * g;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < kOptThreads / 32; ++i) r += sm[i];
    partial[blockIdx.x] = r;
  }
}

// One block: sum the partials in index order, write the norm and the clip scale into the hyper block.
// extra_sumsq (optional) is added: squared norm contributed by other ranks or stages.
__global__ void __launch_bounds__(1024) clip_factor_kernel(const float* __restrict__ partial, int n,
                                                           const float* __restrict__ extra_sumsq,
                                                           float* __restrict__ hyper) {
  __shared__ float sm[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.f;
    for (int i = 0; i < 32; ++i) r += sm[i];
    if (extra_sumsq) r += extra_sumsq[0];
    const float gs = hyper[kHGradScale];
    const float norm = sqrtf(r) * fabsf(gs);
    const float max_norm = hyper[kHMaxNorm];
    float scale = 1.f;
    if (max_norm > 0.f && norm > max_norm) scale = max_norm / (norm + 1e-6f);
    if (!isfinite(norm)) scale = 0.f;   // a non-finite step leaves the weights alone
    hyper[kHGradNorm] = norm;
    hyper[kHClipScale] = scale;
  }
}

__global__ void __launch_bounds__(kOptThreads) multi_adamw_kernel(const OptTensor* __restrict__ tensors,
                                                                  const OptChunk* __restrict__ chunks,
                                                                  const float* __restrict__ hyper, int zero_grad) {
  const OptChunk c = chunks[blockIdx.x];
  const OptTensor t = tensors[c.tensor];
  const long long end = min(t.n, c.first + kOptChunk);
  const float lr = hyper[kHLr], b1 = hyper[kHBeta1], b2 = hyper[kHBeta2], eps = hyper[kHEps];
  const float bc1 = hyper[kHBc1], bc2_sqrt = sqrtf(hyper[kHBc2]);
  const float gscale = hyper[kHClipScale] * hyper[kHGradScale];
  const float decay = 1.f - lr * t.weight_decay;
  const float step_size = lr / bc1;
  for (long long i = c.first + threadIdx.x; i < end; i += kOptThreads) {
    const float g = load_grad(t, i) * gscale;
    float m = t.m[i], v = t.v[i], p = t.master[i];
    m = b1 * m + (1.f - b1) * g;
    v = b2 * v + (1.f - b2) * g * g;
    p *= decay;
    p -= step_size * m / (sqrtf(v) / bc2_sqrt + eps);
    t.m[i] = m;
    t.v[i] = v;
    t.master[i] = p;
    if (t.shadow) t.shadow[i] = __float2bfloat16(p);
    if (zero_grad) {
      if (t.grad_fp32) static_cast<float*>(t.grad)[i] = 0.f;
      else static_cast<__nv_bfloat16*>(t.grad)[i] = __float2bfloat16(0.f);
    }
  }
}

// SGD with momentum on the same tables: buf = mu*buf + g ; p -= lr * (buf + wd*p)
__global__ void __launch_bounds__(kOptThreads) multi_sgd_kernel(const OptTensor* __restrict__ tensors,
                                                                const OptChunk* __restrict__ chunks,
                                                                const float* __restrict__ hyper, float momentum,
                                                                int zero_grad) {
  const OptChunk c = chunks[blockIdx.x];
  const OptTensor t = tensors[c.tensor];
  const long long end = min(t.n, c.first + kOptChunk);
  const float lr = hyper[kHLr];
  const float gscale = hyper[kHClipScale] * hyper[kHGradScale];
  for (long long i = c.first + threadIdx.x; i < end; i += kOptThreads) {
    float p = t.master[i];
    float g = load_grad(t, i) * gscale + t.weight_decay * p;
    if (momentum != 0.f) {
      float b = momentum * t.m[i] + g;
      t.m[i] = b;
      g = b;
    }
    p -= lr * g;
    t.master[i] = p;
    if (t.shadow) t.shadow[i] = __float2bfloat16(p);
    if (zero_grad) {
      if (t.grad_fp32) static_cast<float*>(t.grad)[i] = 0.f;
      else static_cast<__nv_bfloat16*>(t.grad)[i] = __float2bfloat16(0.f);
    }
  }
}

}  // namespace idrak

using namespace idrak;

IDRAK_API int idrak_opt_chunk_elems() { return kOptChunk; }
IDRAK_API int idrak_opt_tensor_bytes() { return int(sizeof(OptTensor)); }
IDRAK_API int idrak_opt_chunk_bytes() { return int(sizeof(OptChunk)); }
IDRAK_API int idrak_opt_hyper_floats() { return kHCount; }

// partial: [n_chunks] floats of scratch. Writes grad norm and clip scale into hyper.
IDRAK_API int idrak_opt_grad_norm(const void* tensors, const void* chunks, int n_chunks, float* partial,
                                  const float* extra_sumsq, float* hyper, void* stream_) {
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  if (n_chunks > 0)
    multi_sumsq_kernel<<<n_chunks, kOptThreads, 0, s>>>(static_cast<const OptTensor*>(tensors),
                                                        static_cast<const OptChunk*>(chunks), partial);
    note_launches(1);
  clip_factor_kernel<<<1, 1024, 0, s>>>(partial, n_chunks, extra_sumsq, hyper);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_opt_adamw(const void* tensors, const void* chunks, int n_chunks, const float* hyper,
                              int zero_grad, void* stream_) {
  if (n_chunks <= 0) return 0;
  multi_adamw_kernel<<<n_chunks, kOptThreads, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const OptTensor*>(tensors), static_cast<const OptChunk*>(chunks), hyper, zero_grad);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_opt_sgd(const void* tensors, const void* chunks, int n_chunks, const float* hyper,
                            float momentum, int zero_grad, void* stream_) {
  if (n_chunks <= 0) return 0;
  multi_sgd_kernel<<<n_chunks, kOptThreads, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const OptTensor*>(tensors), static_cast<const OptChunk*>(chunks), hyper, momentum, zero_grad);
  note_launches(1);
  return int(cudaGetLastError());
}
