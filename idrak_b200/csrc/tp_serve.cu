// Tensor-parallel serving collectives over NVLink peer memory: what a decode or prefill step of a layer-split
// decoder needs between its row-parallel products and the next layer.
//
//   tp_allreduce_rows   one-shot all-reduce of a [rows, dim] bf16 activation held in symmetric buffers, fused with
//                       what follows it in a pre-norm block: out = residual + sum over ranks of their partial
//                       products, and (optionally) normed = RMSNorm / LayerNorm(out) * weight for the next
//                       sub-layer - the reference's "product + residual add + next norm in one launch"
//                       (*_gemv_addnorm_f32, src/Idrak.Gpu/Cuda/PtxKernels.Quantized.cs:454-495) with the sum over
//                       ranks folded in. One block per row; every rank reads all peers' rows and adds them in rank
//                       order, so all ranks hold the same bits and no second exchange is needed.
//   tp_argmax           greedy sampling over a vocabulary split by rows of the head: per-row (value, index) of the
//                       local shard, exchanged through the small-value slots and merged (ties to the lowest index).
//
// Ordering uses one flag channel per call site and a sequence word the kernel advances itself (the last block to
// finish writes it), so a captured CUDA graph replays without any host-side epoch. The caller alternates between
// two symmetric buffers: a rank overwrites a buffer only after it has passed the wait of the following call, by
// which time every peer has finished reading the older one. Waits are bounded and report through the status word.
#include "comm.cuh"

namespace idrak {

struct TpPeerPtrs {
  const __nv_bfloat16* p[kMaxRanks];
};

// Returns true in every thread of the last block to arrive; resets the counter for the next launch.
__device__ __forceinline__ bool tp_last_block(uint32_t* counter) {
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t n = atomicAdd(counter, 1u);
    is_last = (n == gridDim.x - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  return is_last != 0;
}

// One block per row (grid-stride over rows); dim % 8 == 0; blockDim.x * 8 * VPT >= dim.
template <int VPT>
__global__ void __launch_bounds__(512) tp_allreduce_rows_kernel(CommCtx c, TpPeerPtrs bufs, int rows, int dim,
                                                                const __nv_bfloat16* __restrict__ residual,
                                                                __nv_bfloat16* __restrict__ out,
                                                                const __nv_bfloat16* __restrict__ norm_w,
                                                                const __nv_bfloat16* __restrict__ norm_b,
                                                                __nv_bfloat16* __restrict__ normed, float eps,
                                                                int rms, int channel, uint32_t* seq,
                                                                uint32_t* counter) {
  pdl_launch_dependents();     // a dependent launched programmatically may set itself up while this kernel runs
  __shared__ float red[2][16];
  const uint32_t expected = *seq + 1u;
  if (blockIdx.x == 0) signal_peers(c, channel, expected);     // my partial rows are complete (stream order)
  const bool ok = wait_peers(c, channel, expected, 40);
  const int nvec = dim >> 3;
  if (ok) {
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      const size_t base = size_t(row) * dim;
      float v[VPT][8];
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = threadIdx.x + i * blockDim.x;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
        if (vi < nvec) {
          uint4 raw[kMaxRanks];
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p)
            if (p < c.world) raw[p] = ld_peer16(bufs.p[p] + base + vi * 8);
#pragma unroll
          for (int p = 0; p < kMaxRanks; ++p)
            if (p < c.world) accum_bf16x8(v[i], raw[p], 1.f);
          if (residual) {
            const uint4 r = *reinterpret_cast<const uint4*>(residual + base + vi * 8);
            accum_bf16x8(v[i], r, 1.f);
          }
          uint4 o;
          o.x = pack_bf16x2(v[i][0], v[i][1]); o.y = pack_bf16x2(v[i][2], v[i][3]);
          o.z = pack_bf16x2(v[i][4], v[i][5]); o.w = pack_bf16x2(v[i][6], v[i][7]);
          *reinterpret_cast<uint4*>(out + base + vi * 8) = o;
          if (normed) {
            // the norm sees the residual stream as it is stored (bf16), like a separate norm kernel would
            float2 f;
            f = unpack_bf16x2(o.x); v[i][0] = f.x; v[i][1] = f.y;
            f = unpack_bf16x2(o.y); v[i][2] = f.x; v[i][3] = f.y;
            f = unpack_bf16x2(o.z); v[i][4] = f.x; v[i][5] = f.y;
            f = unpack_bf16x2(o.w); v[i][6] = f.x; v[i][7] = f.y;
#pragma unroll
            for (int j = 0; j < 8; ++j) { s1 += v[i][j]; s2 += v[i][j] * v[i][j]; }
          }
        }
      }
      if (normed) {
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s1; red[1][threadIdx.x >> 5] = s2; }
        __syncthreads();
        float t1 = 0.f, t2 = 0.f;
        for (int w = 0; w < int(blockDim.x >> 5); ++w) { t1 += red[0][w]; t2 += red[1][w]; }
        const float mean = rms ? 0.f : t1 / float(dim);
        const float var = rms ? t2 / float(dim) : fmaxf(t2 / float(dim) - mean * mean, 0.f);
        const float rstd = rsqrtf(var + eps);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int vi = threadIdx.x + i * blockDim.x;
          if (vi < nvec) {
            const uint4 wr = *reinterpret_cast<const uint4*>(norm_w + vi * 8);
            float w8[8], b8[8];
            float2 f;
            f = unpack_bf16x2(wr.x); w8[0] = f.x; w8[1] = f.y;
            f = unpack_bf16x2(wr.y); w8[2] = f.x; w8[3] = f.y;
            f = unpack_bf16x2(wr.z); w8[4] = f.x; w8[5] = f.y;
            f = unpack_bf16x2(wr.w); w8[6] = f.x; w8[7] = f.y;
#pragma unroll
            for (int j = 0; j < 8; ++j) b8[j] = 0.f;
            if (norm_b) {
              const uint4 br = *reinterpret_cast<const uint4*>(norm_b + vi * 8);
              f = unpack_bf16x2(br.x); b8[0] = f.x; b8[1] = f.y;
              f = unpack_bf16x2(br.y); b8[2] = f.x; b8[3] = f.y;
              f = unpack_bf16x2(br.z); b8[4] = f.x; b8[5] = f.y;
              f = unpack_bf16x2(br.w); b8[6] = f.x; b8[7] = f.y;
            }
            float n8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) n8[j] = (v[i][j] - mean) * rstd * w8[j] + b8[j];
            uint4 o;
            o.x = pack_bf16x2(n8[0], n8[1]); o.y = pack_bf16x2(n8[2], n8[3]);
            o.z = pack_bf16x2(n8[4], n8[5]); o.w = pack_bf16x2(n8[6], n8[7]);
            *reinterpret_cast<uint4*>(normed + base + vi * 8) = o;
          }
        }
      }
    }
  }
  if (tp_last_block(counter) && threadIdx.x == 0) *seq = expected;
}

// Per row of local logits [rows, ld] (valid columns [0, n_local)): the largest value and its global index
// (offset + column), ties to the lowest column. out: [rows][2] floats (value, index as int bits).
__global__ void __launch_bounds__(1024) tp_argmax_local_kernel(const __nv_bfloat16* __restrict__ logits, int ld,
                                                               int n_local, int offset, float* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* l = logits + size_t(row) * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int j = threadIdx.x; j < n_local; j += blockDim.x) {
    const float v = __bfloat162float(l[j]);
    if (v > best) { best = v; bi = j; }        // ascending j per thread: the first maximum is kept
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
    out[row * 2] = best;
    out[row * 2 + 1] = __int_as_float(bi == 0x7fffffff ? 0x7fffffff : bi + offset);
  }
}

// One block: push this rank's (value, index) pairs into every peer's slots, wait, keep the best per row.
__global__ void __launch_bounds__(256) tp_argmax_merge_kernel(CommCtx c, const float* __restrict__ local, int rows,
                                                              int* __restrict__ ids, int channel, uint32_t* seq) {
  const uint32_t expected = *seq + 1u;
  for (int i = threadIdx.x; i < rows * 2 * c.world; i += blockDim.x) {
    const int p = i / (rows * 2), k = i - p * rows * 2;
    c.slots[p][c.rank * c.slot_floats + k] = local[k];
  }
  __syncthreads();
  signal_peers(c, channel, expected);
  if (wait_peers(c, channel, expected, 41)) {
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int p = 0; p < c.world; ++p) {
        const float v = __ldcg(c.slots[c.rank] + p * c.slot_floats + r * 2);
        const int idx = __float_as_int(__ldcg(c.slots[c.rank] + p * c.slot_floats + r * 2 + 1));
        if (v > best || (v == best && idx < bi)) { best = v; bi = idx; }
      }
      ids[r] = bi;
    }
  }
  // the slots may be rewritten once every rank has read them
  __syncthreads();
  signal_peers(c, channel + 1, expected);
  wait_peers(c, channel + 1, expected, 42);
  __syncthreads();
  if (threadIdx.x == 0) *seq = expected;
}

}  // namespace idrak

using namespace idrak;

static inline CommCtx tp_load_ctx(const void* ctx) {
  CommCtx c;
  memcpy(&c, ctx, sizeof(c));
  return c;
}

// out[rows, dim] = residual + sum over ranks of bufs[p][rows, dim]; normed = norm(out) * norm_w (+ norm_b) when
// `normed` is given. `seq` and `counter` are two device words owned by the call site (zero at start).
IDRAK_API int idrak_tp_allreduce_rows(const void* ctx, void* const* bufs, int rows, int dim, const void* residual,
                                      void* out, const void* norm_w, const void* norm_b, void* normed, float eps,
                                      int rms, int channel, void* seq, void* counter, void* stream_) {
  if (rows <= 0) return 0;
  if (dim % 8 || dim > 8 * 512 * 4) return -2;
  if (channel < 0 || channel + 1 >= kFlagChannels) return -3;
  if (normed && !norm_w) return -4;
  CommCtx c = tp_load_ctx(ctx);
  TpPeerPtrs p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < c.world && i < kMaxRanks; ++i) p.p[i] = static_cast<const __nv_bfloat16*>(bufs[i]);
  const int nvec = dim / 8;
  int threads = 32;
  while (threads < 512 && threads < nvec) threads *= 2;
  const int vpt = (nvec + threads - 1) / threads;
  const int grid = rows < 4 * sm_count() ? rows : 4 * sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
#define IDRAK_TP_AR(V)                                                                                              \
  tp_allreduce_rows_kernel<V><<<grid, threads, 0, s>>>(                                                             \
      c, p, rows, dim, static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out),              \
      static_cast<const __nv_bfloat16*>(norm_w), static_cast<const __nv_bfloat16*>(norm_b),                        \
      static_cast<__nv_bfloat16*>(normed), eps, rms, channel, static_cast<uint32_t*>(seq),                         \
      static_cast<uint32_t*>(counter))
  if (vpt <= 1) IDRAK_TP_AR(1);
  else if (vpt <= 2) IDRAK_TP_AR(2);
  else IDRAK_TP_AR(4);
#undef IDRAK_TP_AR
  note_launches(1);
  return int(cudaGetLastError());
}

// ids[rows] = index of the largest logit over all ranks' shards. `local` holds rows * 2 floats of scratch.
IDRAK_API int idrak_tp_argmax(const void* ctx, const void* logits, int ld, int rows, int n_local, int offset,
                              float* local, int* ids, int channel, void* seq, void* stream_) {
  if (rows <= 0) return 0;
  CommCtx c = tp_load_ctx(ctx);
  if (rows * 2 > c.slot_floats) return -2;
  if (channel < 0 || channel + 1 >= kFlagChannels) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  tp_argmax_local_kernel<<<rows, 1024, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), ld, n_local, offset, local);
  tp_argmax_merge_kernel<<<1, 256, 0, s>>>(c, local, rows, ids, channel, static_cast<uint32_t*>(seq));
  note_launches(2);
  return int(cudaGetLastError());
}
