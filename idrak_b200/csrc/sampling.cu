// Device-side token sampling over logits rows: greedy arg-max, and temperature / top-k / top-p / min-p
// sampling with repetition, presence and frequency penalties. One block per row; the host reads the chosen
// ids (one int per row), never the logits.
//
// sample_rows_kernel: (1) penalties and temperature are applied on the fly; (2) the k-th largest value is
// found with a 4-pass radix select over the order-preserving integer image of the floats (shared-memory
// histograms, no sort of the vocabulary); (3) the <= 64 survivors are gathered, sorted by value (ties: lower id
// first) in shared memory, soft-maxed, cut by top-p / min-p, and one is drawn with a counter-based hash of
// (seed, row, step) so a run repeats exactly.
//
// Reference counterparts: sample_rows_f32, sample_candidates(_greedy)_f32, topk_candidates_f32, topk_greedy_f32
// (CandidateSlots = 64), penalize_rows_f32 (src/Idrak.Gpu/Cuda/PtxKernels.Decoding.cs:12), SamplingSettings /
// TokenSampler (src/Idrak.Abstraction/Generation/SamplingSettings.cs, TokenSamplers.cs).
#include "common.cuh"

namespace idrak {

constexpr int kSampleThreads = 1024;
constexpr int kCandidates = 64;

__device__ __forceinline__ float load_logit(const void* base, int fp32, size_t i) {
  return fp32 ? static_cast<const float*>(base)[i] : __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]);
}
__device__ __forceinline__ uint32_t ordered_bits(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

// ids[row] = argmax_j logits[row, j] (lowest index among ties)
__global__ void __launch_bounds__(kSampleThreads) argmax_rows_kernel(const void* __restrict__ logits, int fp32,
                                                                     int vocab, long long ld, int* __restrict__ ids) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  int tail_from = 0;
  if (!fp32 && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    // bf16 rows that start on 16 bytes: eight logits per load
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(logits) + size_t(row) * ld);
    const int nvec = vocab >> 3;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      const uint4 u = src[c];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float lo = __uint_as_float(w[h] << 16), hi = __uint_as_float(w[h] & 0xffff0000u);
        const int j = c * 8 + h * 2;
        if (lo > best || (lo == best && j < bi)) { best = lo; bi = j; }
        if (hi > best || (hi == best && j + 1 < bi)) { best = hi; bi = j + 1; }
      }
    }
    tail_from = nvec << 3;
  }
  for (int j = tail_from + threadIdx.x; j < vocab; j += blockDim.x) {
    const float v = load_logit(logits, fp32, size_t(row) * ld + j);
    if (v > best || (v == best && j < bi)) { best = v; bi = j; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < int(blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    ids[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

struct SampleParams {
  const void* logits;
  int fp32, vocab;
  long long ld;
  int* ids;                    // out [rows]
  float* logprobs;             // out [rows] log-probability of the chosen token under the final distribution, or null
  const float* temperature;    // per row
  const int* top_k;            // per row (<= 0: 64)
  const float* top_p;          // per row
  const float* min_p;          // per row
  const int* history;          // [rows, history_len] recent token ids (-1 = empty) or null
  int history_len;
  const float* repeat_penalty; // per row (1 = off)
  const float* presence_penalty;
  const float* frequency_penalty;
  const unsigned long long* seeds;   // per row
  unsigned step;
};

__device__ __forceinline__ float penalised(const SampleParams& p, int row, int j, float v) {
  if (p.history == nullptr) return v;
  int count = 0;
  const int* h = p.history + size_t(row) * p.history_len;
  for (int i = 0; i < p.history_len; ++i) count += (h[i] == j);
  if (count == 0) return v;
  const float rp = p.repeat_penalty ? p.repeat_penalty[row] : 1.f;
  if (rp != 1.f) v = v > 0.f ? v / rp : v * rp;
  if (p.presence_penalty) v -= p.presence_penalty[row];
  if (p.frequency_penalty) v -= p.frequency_penalty[row] * float(count);
  return v;
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(const SampleParams p) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_remaining;
  __shared__ float cand_v[kCandidates * 2];
  __shared__ int cand_i[kCandidates * 2];
  __shared__ int n_cand;
  __shared__ int tie_warp[32];
  const int row = blockIdx.x;
  const float temp = fmaxf(p.temperature ? p.temperature[row] : 1.f, 1e-6f);
  int k = p.top_k ? p.top_k[row] : kCandidates;
  if (k <= 0 || k > kCandidates) k = kCandidates;
  if (k > p.vocab) k = p.vocab;

  // ---- radix select: the order-preserving bits of the k-th largest value
  if (threadIdx.x == 0) { s_prefix = 0; s_remaining = uint32_t(k); }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int j = threadIdx.x; j < p.vocab; j += blockDim.x) {
      const float v = penalised(p, row, j, load_logit(p.logits, p.fp32, size_t(row) * p.ld + j)) / temp;
      const uint32_t b = ordered_bits(v);
      if ((b & mask) == prefix) atomicAdd(&hist[(b >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t remaining = s_remaining, digit = 0;
      for (int d = 255; d >= 0; --d) {
        if (hist[d] >= remaining) { digit = uint32_t(d); break; }
        remaining -= hist[d];
      }
      s_prefix = prefix | (digit << shift);
      s_remaining = remaining;
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;
  // ---- gather candidates: everything strictly above the k-th value (fewer than k of them, in any order: they are
  // sorted below), then as many entries equal to it as the k places still need, by ascending id. Ties can never
  // crowd a larger logit out of the slots, and which tied ids are kept does not depend on thread timing.
  if (threadIdx.x == 0) n_cand = 0;
  __syncthreads();
  for (int j = threadIdx.x; j < p.vocab; j += blockDim.x) {
    const float v = penalised(p, row, j, load_logit(p.logits, p.fp32, size_t(row) * p.ld + j)) / temp;
    if (ordered_bits(v) > kth) {
      const int slot = atomicAdd(&n_cand, 1);
      if (slot < kCandidates * 2) { cand_v[slot] = v; cand_i[slot] = j; }
    }
  }
  __syncthreads();
  {
    const int n_greater = min(n_cand, kCandidates * 2);
    const int need = min(k - n_greater, kCandidates * 2 - n_greater);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    int tie_base = 0;
    for (int base = 0; base < p.vocab && tie_base < need; base += blockDim.x) {
      const int j = base + threadIdx.x;
      float v = 0.f;
      bool tie = false;
      if (j < p.vocab) {
        v = penalised(p, row, j, load_logit(p.logits, p.fp32, size_t(row) * p.ld + j)) / temp;
        tie = ordered_bits(v) == kth;
      }
      const unsigned ballot = __ballot_sync(0xffffffffu, tie);
      if (lane == 0) tie_warp[warp] = __popc(ballot);
      __syncthreads();
      int before = 0, total = 0;
      for (int w = 0; w < warps; ++w) {
        const int c = tie_warp[w];
        if (w < warp) before += c;
        total += c;
      }
      if (tie) {
        const int pos = tie_base + before + __popc(ballot & ((1u << lane) - 1u));
        if (pos < need) { cand_v[n_greater + pos] = v; cand_i[n_greater + pos] = j; }
      }
      tie_base += total;
      __syncthreads();
    }
    if (threadIdx.x == 0) n_cand = n_greater + max(0, min(tie_base, need));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = min(n_cand, kCandidates * 2);
    // insertion sort: value descending, id ascending (n <= 128)
    for (int a = 1; a < n; ++a) {
      const float v = cand_v[a];
      const int id = cand_i[a];
      int b = a - 1;
      while (b >= 0 && (cand_v[b] < v || (cand_v[b] == v && cand_i[b] > id))) {
        cand_v[b + 1] = cand_v[b];
        cand_i[b + 1] = cand_i[b];
        --b;
      }
      cand_v[b + 1] = v;
      cand_i[b + 1] = id;
    }
    n = min(n, k);
    const float mx = cand_v[0];
    float total = 0.f;
    for (int a = 0; a < n; ++a) { cand_v[a] = __expf(cand_v[a] - mx); total += cand_v[a]; }
    // min-p then top-p on the sorted probabilities
    const float minp = p.min_p ? p.min_p[row] : 0.f;
    const float topp = p.top_p ? p.top_p[row] : 1.f;
    int keep = n;
    if (minp > 0.f) {
      keep = 0;
      while (keep < n && cand_v[keep] >= minp * cand_v[0]) ++keep;
      keep = max(keep, 1);
    }
    if (topp < 1.f) {
      float cum = 0.f;
      int c = 0;
      while (c < keep) {
        cum += cand_v[c] / total;
        ++c;
        if (cum >= topp) break;
      }
      keep = max(c, 1);
    }
    float kept = 0.f;
    for (int a = 0; a < keep; ++a) kept += cand_v[a];
    const unsigned long long seed = p.seeds ? p.seeds[row] : 0ull;
    // the draw depends on the row's seed and the step only, never on where the row sits in the batch
    uint32_t r = hash32(uint32_t(seed) ^ hash32(uint32_t(seed >> 32) + 0x9e3779b9u * (p.step + 1u)));
    const float u = (float(r >> 8) + 0.5f) * (1.0f / 16777216.0f) * kept;
    float cum = 0.f;
    int pick = keep - 1;
    for (int a = 0; a < keep; ++a) {
      cum += cand_v[a];
      if (u < cum) { pick = a; break; }
    }
    p.ids[row] = cand_i[pick];
    if (p.logprobs) p.logprobs[row] = __logf(cand_v[pick] / kept);
  }
}

}  // namespace idrak

using namespace idrak;

IDRAK_API int idrak_argmax_rows(const void* logits, int fp32, int rows, int vocab, long long ld, int* ids,
                                void* stream_) {
  if (rows <= 0) return 0;
  argmax_rows_kernel<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream_)>>>(logits, fp32, vocab, ld, ids);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_sample_rows(const void* logits, int fp32, int rows, int vocab, long long ld, int* ids,
                                float* logprobs, const float* temperature, const int* top_k, const float* top_p,
                                const float* min_p, const int* history, int history_len, const float* repeat_penalty,
                                const float* presence_penalty, const float* frequency_penalty,
                                const unsigned long long* seeds, unsigned step, void* stream_) {
  if (rows <= 0) return 0;
  SampleParams p;
  p.logits = logits; p.fp32 = fp32; p.vocab = vocab; p.ld = ld; p.ids = ids; p.logprobs = logprobs;
  p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.min_p = min_p;
  p.history = history; p.history_len = history_len;
  p.repeat_penalty = repeat_penalty; p.presence_penalty = presence_penalty; p.frequency_penalty = frequency_penalty;
  p.seeds = seeds; p.step = step;
  sample_rows_kernel<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream_)>>>(p);
  note_launches(1);
  return int(cudaGetLastError());
}
