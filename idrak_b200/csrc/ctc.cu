// Connectionist temporal classification loss: forward (alpha recursion) and backward (beta recursion + gradient with
// respect to the log-probabilities), in the log domain, one CTA per sequence, threads over the positions of the
// extended label string (blank, l1, blank, l2, ... blank).
//
// A time step needs the previous row of the recursion only, so two rows ping-pong in shared memory when the extended
// string fits (6000 positions, just under 48 KB) and in a global scratch otherwise; the alpha rows are also written to global
// memory because the backward pass reads them. The gradient of class c at time t is a sum over the positions that carry
// c: blanks (every even position) by a block reduction, labels by a chain built once per sequence that links the
// positions of equal labels in ascending order, so the sum runs in a fixed order and reruns agree bit for bit.
//
// Reference counterparts: ctc_loss_f32 / ctc_loss_global_f32 / ctc_loss_bwd_f32 / ctc_loss_bwd_global_f32
// (src/Idrak.Gpu/Cuda/PtxKernels.Ctc.cs).
#include "common.cuh"
#include <cfloat>

namespace idrak {

constexpr int kCtcThreads = 256;
constexpr int kCtcSmemPositions = 6000;      // two fp32 rows of this many positions stay under 48 KB
constexpr float kNegInf = -1e30f;            // stands for log(0); finite so that differences stay finite

__device__ __forceinline__ float log_add(float a, float b) {
  const float m = fmaxf(a, b);
  if (m <= kNegInf) return kNegInf;
  return m + __logf(__expf(a - m) + __expf(b - m));
}
__device__ __forceinline__ float log_add3(float a, float b, float c) {
  const float m = fmaxf(a, fmaxf(b, c));
  if (m <= kNegInf) return kNegInf;
  return m + __logf(__expf(a - m) + __expf(b - m) + __expf(c - m));
}

// log_probs [T, B, C]; targets [B, max_target]; alpha [B, T, S] with S = 2 * max_target + 1; loss [B].
// rows: scratch [B, 2, S], used when S > kCtcSmemPositions.
__global__ void __launch_bounds__(kCtcThreads) ctc_alpha_kernel(const float* __restrict__ log_probs,
                                                                const int* __restrict__ targets,
                                                                const int* __restrict__ input_lengths,
                                                                const int* __restrict__ target_lengths,
                                                                float* __restrict__ alpha, float* __restrict__ rows,
                                                                float* __restrict__ loss, int T, int B, int C,
                                                                int max_target, int blank, int use_smem) {
  extern __shared__ float smem[];
  const int b = blockIdx.x;
  const int S_all = 2 * max_target + 1;
  const int L = min(target_lengths[b], max_target);
  const int S = 2 * L + 1;
  const int Tb = min(input_lengths[b], T);
  float* row[2];
  row[0] = use_smem ? smem : rows + (size_t(b) * 2) * S_all;
  row[1] = row[0] + S_all;
  const int* tg = targets + size_t(b) * max_target;
  float* ab = alpha + size_t(b) * T * S_all;
  if (Tb < 1) {
    if (threadIdx.x == 0) loss[b] = L == 0 ? 0.f : FLT_MAX;
    return;
  }
  // t = 0: only the first blank and the first label can start a path
  const float* lp0 = log_probs + size_t(b) * C;
  for (int s = threadIdx.x; s < S_all; s += blockDim.x) {
    float v = kNegInf;
    if (s == 0) v = lp0[blank];
    else if (s == 1 && L > 0) v = lp0[tg[0]];
    row[0][s] = v;
    ab[s] = v;
  }
  __syncthreads();
  for (int t = 1; t < Tb; ++t) {
    const float* lp = log_probs + (size_t(t) * B + b) * C;
    const float* prev = row[(t - 1) & 1];
    float* cur = row[t & 1];
    for (int s = threadIdx.x; s < S_all; s += blockDim.x) {
      float v = kNegInf;
      if (s < S) {
        const int cls = (s & 1) ? tg[s >> 1] : blank;
        const float a0 = prev[s];
        const float a1 = s >= 1 ? prev[s - 1] : kNegInf;
        const float a2 = (s >= 2 && (s & 1) && tg[s >> 1] != tg[(s >> 1) - 1]) ? prev[s - 2] : kNegInf;
        const float m = log_add3(a0, a1, a2);
        v = m <= kNegInf ? kNegInf : m + lp[cls];
      }
      cur[s] = v;
      ab[size_t(t) * S_all + s] = v;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float* last = row[(Tb - 1) & 1];
    const float tot = log_add(last[S - 1], S >= 2 ? last[S - 2] : kNegInf);
    loss[b] = tot <= kNegInf ? FLT_MAX : -tot;          // FLT_MAX: no alignment exists
  }
}

// grad [T, B, C] must be zero on entry. grad_out [B] scales each sequence's gradient. `chain` [B, S] int scratch.
__global__ void __launch_bounds__(kCtcThreads) ctc_beta_kernel(const float* __restrict__ log_probs,
                                                               const int* __restrict__ targets,
                                                               const int* __restrict__ input_lengths,
                                                               const int* __restrict__ target_lengths,
                                                               const float* __restrict__ alpha,
                                                               const float* __restrict__ loss,
                                                               const float* __restrict__ grad_out,
                                                               float* __restrict__ rows, int* __restrict__ chain,
                                                               float* __restrict__ grad, int T, int B, int C,
                                                               int max_target, int blank, int use_smem) {
  extern __shared__ float smem[];
  __shared__ float scratch[kCtcThreads / 32];
  const int b = blockIdx.x;
  const int S_all = 2 * max_target + 1;
  const int L = min(target_lengths[b], max_target);
  const int S = 2 * L + 1;
  const int Tb = min(input_lengths[b], T);
  const float nll = loss[b];
  if (Tb < 1 || nll >= FLT_MAX) return;                 // no alignment: the gradient stays zero
  const float go = grad_out ? grad_out[b] : 1.f;
  float* row[2];
  row[0] = use_smem ? smem : rows + (size_t(b) * 2) * S_all;
  row[1] = row[0] + S_all;
  const int* tg = targets + size_t(b) * max_target;
  const float* ab = alpha + size_t(b) * T * S_all;
  int* next = chain + size_t(b) * S_all;
  // chain of equal labels: next[s] = the next odd position with the same label (0 = none); next[s] < 0 marks a position
  // that is not the first of its label (-1 - next). Position s = 2 i + 1 carries label i.
  for (int i = threadIdx.x; i < L; i += blockDim.x) {
    const int lab = tg[i];
    int nx = 0;
    for (int j = i + 1; j < L; ++j)
      if (tg[j] == lab) { nx = 2 * j + 1; break; }
    bool first = true;
    for (int j = 0; j < i; ++j)
      if (tg[j] == lab) { first = false; break; }
    next[2 * i + 1] = first ? nx : -1 - nx;
  }
  // t = Tb - 1: a path may end in the last blank or the last label
  {
    const float* lp = log_probs + (size_t(Tb - 1) * B + b) * C;
    float* cur = row[(Tb - 1) & 1];
    for (int s = threadIdx.x; s < S_all; s += blockDim.x) {
      float v = kNegInf;
      if (s == S - 1) v = lp[blank];
      else if (s == S - 2 && L > 0) v = lp[tg[L - 1]];
      cur[s] = v;
    }
  }
  __syncthreads();
  for (int t = Tb - 1; t >= 0; --t) {
    const float* lp = log_probs + (size_t(t) * B + b) * C;
    float* g = grad + (size_t(t) * B + b) * C;
    float* cur = row[t & 1];
    const float* at = ab + size_t(t) * S_all;
    // blanks: log-sum over the even positions, by block reductions
    float m = kNegInf;
    for (int s = 2 * threadIdx.x; s < S; s += 2 * blockDim.x) m = fmaxf(m, at[s] + cur[s]);
    m = warp_max(m);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
    __syncthreads();
    m = scratch[0];
    for (int w = 1; w < kCtcThreads / 32; ++w) m = fmaxf(m, scratch[w]);
    float sum = 0.f;
    if (m > kNegInf)
      for (int s = 2 * threadIdx.x; s < S; s += 2 * blockDim.x) sum += __expf(at[s] + cur[s] - m);
    sum = warp_sum(sum);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0 && m > kNegInf) {
      float tot = 0.f;
      for (int w = 0; w < kCtcThreads / 32; ++w) tot += scratch[w];
      g[blank] = -go * __expf(m + __logf(tot) - lp[blank] + nll);
    }
    // labels: the first position of each label walks its chain
    for (int s = 2 * threadIdx.x + 1; s < S; s += 2 * blockDim.x) {
      int nx = next[s];
      if (nx < 0) continue;
      float mm = at[s] + cur[s];
      for (int p = nx; p > 0; p = -1 - next[p]) mm = fmaxf(mm, at[p] + cur[p]);
      if (mm <= kNegInf) continue;
      float acc = __expf(at[s] + cur[s] - mm);
      for (int p = nx; p > 0; p = -1 - next[p]) acc += __expf(at[p] + cur[p] - mm);
      const int cls = tg[s >> 1];
      g[cls] = -go * __expf(mm + __logf(acc) - lp[cls] + nll);
    }
    // beta of t - 1
    if (t > 0) {
      const float* lpp = log_probs + (size_t(t - 1) * B + b) * C;
      float* prv = row[(t - 1) & 1];
      for (int s = threadIdx.x; s < S_all; s += blockDim.x) {
        float v = kNegInf;
        if (s < S) {
          const int cls = (s & 1) ? tg[s >> 1] : blank;
          const float b0 = cur[s];
          const float b1 = s + 1 < S ? cur[s + 1] : kNegInf;
          const float b2 = (s + 2 < S && (s & 1) && tg[s >> 1] != tg[(s >> 1) + 1]) ? cur[s + 2] : kNegInf;
          const float mm = log_add3(b0, b1, b2);
          v = mm <= kNegInf ? kNegInf : mm + lpp[cls];
        }
        prv[s] = v;
      }
    }
    __syncthreads();
  }
}

}  // namespace idrak

using namespace idrak;

// Floats of scratch the two calls need: alpha [B, T, S] and rows [B, 2, S]; the chain takes B * S ints.
IDRAK_API long long idrak_ctc_alpha_elems(int T, int B, int max_target) {
  return (long long)B * T * (2 * max_target + 1);
}
IDRAK_API long long idrak_ctc_row_elems(int B, int max_target) { return (long long)B * 2 * (2 * max_target + 1); }

IDRAK_API int idrak_ctc_loss(const float* log_probs, const int* targets, const int* input_lengths,
                             const int* target_lengths, float* alpha, float* rows, float* loss, int T, int B, int C,
                             int max_target, int blank, void* stream_) {
  if (T < 1 || B < 1 || C < 1 || max_target < 0 || blank < 0 || blank >= C) return -2;
  const int S = 2 * max_target + 1;
  const int use_smem = S <= kCtcSmemPositions;
  const size_t smem = use_smem ? size_t(2) * S * sizeof(float) : 0;
  ctc_alpha_kernel<<<B, kCtcThreads, smem, static_cast<cudaStream_t>(stream_)>>>(
      log_probs, targets, input_lengths, target_lengths, alpha, rows, loss, T, B, C, max_target, blank, use_smem);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_ctc_loss_bwd(const float* log_probs, const int* targets, const int* input_lengths,
                                 const int* target_lengths, const float* alpha, const float* loss,
                                 const float* grad_out, float* rows, int* chain, float* grad, int T, int B, int C,
                                 int max_target, int blank, void* stream_) {
  if (T < 1 || B < 1 || C < 1 || max_target < 0 || blank < 0 || blank >= C) return -2;
  const int S = 2 * max_target + 1;
  const int use_smem = S <= kCtcSmemPositions;
  const size_t smem = use_smem ? size_t(2) * S * sizeof(float) : 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  cudaError_t e = cudaMemsetAsync(grad, 0, size_t(T) * B * C * sizeof(float), stream);
  if (e != cudaSuccess) return int(e);
  e = cudaMemsetAsync(chain, 0, size_t(B) * S * sizeof(int), stream);
  if (e != cudaSuccess) return int(e);
  ctc_beta_kernel<<<B, kCtcThreads, smem, stream>>>(log_probs, targets, input_lengths, target_lengths, alpha, loss,
                                                    grad_out, rows, chain, grad, T, B, C, max_target, blank, use_smem);
  note_launches(1);
  return int(cudaGetLastError());
}
