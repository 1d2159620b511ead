// Fused softmax cross-entropy over bf16 logits: one block per row reads the row once into registers,
// computes the loss and overwrites the logits with their gradient (softmax - onehot) * scale.
// Columns at and beyond `vocab` (padding up to the row stride) get gradient 0 and take no part in the
// softmax. Rows whose target is `ignore_index` get loss 0 and gradient 0.
//
// Reference counterpart: softmax_ce_rows_f32, "loss + in-place logits -> gradient, one block per row"
// (src/Idrak.Gpu/Cuda/PtxKernels.Decoder.cs:12,75-77) driven by Tensor.TokenCrossEntropy
// (src/Idrak.Abstraction/Tensors/Tensor.Decoder.cs:73) so the caller can run the head in row chunks.
#include "common.cuh"

namespace idrak {

constexpr int kXentThreads = 1024;
constexpr int kXentMaxVec = 8;   // 8 x 8 bf16 per thread -> rows up to 65,536 columns stay in registers

__device__ __forceinline__ float block_reduce(float v, float* sm, bool is_max) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) sm[wid] = v;
  __syncthreads();
  float r = sm[0];
  const int warps = blockDim.x >> 5;
  for (int i = 1; i < warps; ++i) r = is_max ? fmaxf(r, sm[i]) : r + sm[i];   // same order in every thread
  return r;
}

template <int NV>
__global__ void __launch_bounds__(kXentThreads) xent_kernel(__nv_bfloat16* __restrict__ logits,
                                                            const int* __restrict__ targets,
                                                            float* __restrict__ losses, float* __restrict__ lse_out,
                                                            int vocab, int ld, float scale, int ignore_index,
                                                            int write_grad) {
  __shared__ float sm[32];
  const int row = blockIdx.x;
  __nv_bfloat16* lrow = logits + size_t(row) * ld;
  const int target = targets[row];
  const int nvec = ld >> 3;   // whole row stride: padding columns get gradient 0
  uint4 raw[NV];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kXentThreads;
    if (vi < nvec) {
      raw[i] = *reinterpret_cast<const uint4*>(lrow + vi * 8);
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = unpack_bf16x2(w[k]);
        const int c = vi * 8 + k * 2;
        if (c < vocab) mx = fmaxf(mx, f.x);
        if (c + 1 < vocab) mx = fmaxf(mx, f.y);
      }
    }
  }
  mx = block_reduce(mx, sm, true);
  float se = 0.f;
  const float l2e = 1.4426950408889634f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kXentThreads;
    if (vi < nvec) {
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = unpack_bf16x2(w[k]);
        const int c = vi * 8 + k * 2;
        if (c < vocab) se += exp2f((f.x - mx) * l2e);
        if (c + 1 < vocab) se += exp2f((f.y - mx) * l2e);
      }
    }
  }
  se = block_reduce(se, sm, false);
  const float lse = mx + logf(se);
  const bool ignored = (target == ignore_index) || target < 0 || target >= vocab;
  if (threadIdx.x == 0) {
    const float lt = ignored ? 0.f : __bfloat162float(lrow[target]);
    losses[row] = ignored ? 0.f : (lse - lt);
    if (lse_out) lse_out[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();   // thread 0 has read lrow[target] before anyone overwrites it
  const float inv = ignored ? 0.f : scale / se;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * kXentThreads;
    if (vi < nvec) {
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = unpack_bf16x2(w[k]);
        const int c = vi * 8 + k * 2;
        float g0 = (c < vocab) ? exp2f((f.x - mx) * l2e) * inv : 0.f;
        float g1 = (c + 1 < vocab) ? exp2f((f.y - mx) * l2e) * inv : 0.f;
        if (!ignored) {
          if (c == target) g0 -= scale;
          if (c + 1 == target) g1 -= scale;
        }
        o[k] = pack_bf16x2(g0, g1);
      }
      *reinterpret_cast<uint4*>(lrow + vi * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Rows too wide for registers: same arithmetic, the row is read from memory in each of the three passes
// (the second and third mostly hit L2).
__global__ void __launch_bounds__(kXentThreads) xent_stream_kernel(__nv_bfloat16* __restrict__ logits,
                                                                   const int* __restrict__ targets,
                                                                   float* __restrict__ losses,
                                                                   float* __restrict__ lse_out, int vocab, int ld,
                                                                   float scale, int ignore_index, int write_grad) {
  __shared__ float sm[32];
  const int row = blockIdx.x;
  __nv_bfloat16* lrow = logits + size_t(row) * ld;
  const int target = targets[row];
  const int nvec = ld >> 3;
  const float l2e = 1.4426950408889634f;
  float mx = -INFINITY;
  for (int vi = threadIdx.x; vi < nvec; vi += kXentThreads) {
    uint4 r = *reinterpret_cast<const uint4*>(lrow + vi * 8);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = unpack_bf16x2(w[k]);
      const int c = vi * 8 + k * 2;
      if (c < vocab) mx = fmaxf(mx, f.x);
      if (c + 1 < vocab) mx = fmaxf(mx, f.y);
    }
  }
  mx = block_reduce(mx, sm, true);
  float se = 0.f;
  for (int vi = threadIdx.x; vi < nvec; vi += kXentThreads) {
    uint4 r = *reinterpret_cast<const uint4*>(lrow + vi * 8);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = unpack_bf16x2(w[k]);
      const int c = vi * 8 + k * 2;
      if (c < vocab) se += exp2f((f.x - mx) * l2e);
      if (c + 1 < vocab) se += exp2f((f.y - mx) * l2e);
    }
  }
  se = block_reduce(se, sm, false);
  const float lse = mx + logf(se);
  const bool ignored = (target == ignore_index) || target < 0 || target >= vocab;
  if (threadIdx.x == 0) {
    const float lt = ignored ? 0.f : __bfloat162float(lrow[target]);
    losses[row] = ignored ? 0.f : (lse - lt);
    if (lse_out) lse_out[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();
  const float inv = ignored ? 0.f : scale / se;
  for (int vi = threadIdx.x; vi < nvec; vi += kXentThreads) {
    uint4 r = *reinterpret_cast<const uint4*>(lrow + vi * 8);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = unpack_bf16x2(w[k]);
      const int c = vi * 8 + k * 2;
      float g0 = (c < vocab) ? exp2f((f.x - mx) * l2e) * inv : 0.f;
      float g1 = (c + 1 < vocab) ? exp2f((f.y - mx) * l2e) * inv : 0.f;
      if (!ignored) {
        if (c == target) g0 -= scale;
        if (c + 1 == target) g1 -= scale;
      }
      o[k] = pack_bf16x2(g0, g1);
    }
    *reinterpret_cast<uint4*>(lrow + vi * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// out[0] = sum(losses) * scale, summed in index order by one block (deterministic).
__global__ void __launch_bounds__(1024) sum_rows_kernel(const float* __restrict__ v, int n, float scale,
                                                        float* __restrict__ out) {
  __shared__ float sm[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += v[i];
  s = block_reduce(s, sm, false);
  if (threadIdx.x == 0) out[0] = s * scale;
}

// xent_bulk.cu: the pipelined kernel for rows that fit shared memory twice; -100 = sizes do not fit.
int xent_bulk_launch(void* logits, const int* targets, float* losses, float* lse, int rows, int vocab, int ld,
                     float scale, int ignore_index, int write_grad, cudaStream_t stream);

}  // namespace idrak

using namespace idrak;

// logits: [rows, ld] bf16 with ld % 8 == 0 and ld >= round_up(vocab, 8). In place -> gradient when write_grad.
IDRAK_API int idrak_softmax_xent(void* logits, const int* targets, float* losses, float* lse, int rows, int vocab,
                                 int ld, float scale, int ignore_index, int write_grad, void* stream_) {
  if (ld % 8 || ld < ((vocab + 7) / 8) * 8) return -2;
  const int nvec = ld / 8;
  const int nv = (nvec + kXentThreads - 1) / kXentThreads;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  __nv_bfloat16* l = static_cast<__nv_bfloat16*>(logits);
  {
    const int rc = xent_bulk_launch(logits, targets, losses, lse, rows, vocab, ld, scale, ignore_index, write_grad, s);
    if (rc != -100) return rc;
  }
  if (nv > kXentMaxVec) {
    xent_stream_kernel<<<rows, kXentThreads, 0, s>>>(l, targets, losses, lse, vocab, ld, scale, ignore_index, write_grad);
    note_launches(1);
    return int(cudaGetLastError());
  }
#define XE(V) xent_kernel<V><<<rows, kXentThreads, 0, s>>>(l, targets, losses, lse, vocab, ld, scale, ignore_index, write_grad)
  switch (nv) {
    case 1: XE(1); break;
    case 2: XE(2); break;
    case 3: XE(3); break;
    case 4: XE(4); break;
    case 5: XE(5); break;
    case 6: XE(6); break;
    case 7: XE(7); break;
    default: XE(8); break;
  }
#undef XE
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_sum_rows(const float* v, int n, float scale, float* out, void* stream_) {
  sum_rows_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream_)>>>(v, n, scale, out);
  note_launches(1);
  return int(cudaGetLastError());
}
