// Collectives over NVLink peer memory, written as kernels that issue the peer loads and stores themselves,
// and the fused data-parallel step built from them.
//
// Plumbing: every rank owns "symmetric" buffers (same size on every rank) allocated here with cudaMalloc and
// shared through CUDA IPC handles; a kernel receives a table of the W peer pointers. Ordering between ranks
// uses flag words in symmetric memory: a writer stores a monotone epoch into slot [channel][writer] of every
// peer's flag area (st.release.sys after a system fence); a reader polls its own copy (ld.acquire.sys).
// Every poll is bounded (two seconds): on expiry the kernel records (code, channel, peer rank) in the
// host-visible status word and returns, so a missing peer ends as a Python exception that names the rank,
// never as a hung GPU.
//
// Kernels
//   allreduce_oneshot      small float vectors (headers, norms, stop flags): every rank writes its values into
//                          every peer, then sums the W copies in rank order.
//   allreduce_twoshot      bf16 / fp32 vectors: reduce-scatter by peer loads (each rank sums its 1/W slice in
//                          fixed rank order), then all-gather by peer stores.
//   reduce_scatter / all_gather / broadcast
//   dp_reduce_scatter      per gradient bucket: wait for the peers' bucket, sum the W bf16 gradients of this
//                          rank's slice in rank order (optionally token-weighted), keep the fp32 result as the
//                          shard gradient and emit partial sums of squares for the global norm.
//   dp_norm_exchange       global gradient norm over all ranks -> clip scale (one-shot exchange).
//   dp_adamw_allgather     AdamW on the rank's shard (fp32 master + moments) fused with the all-gather: the new
//                          bf16 weights are stored straight into every peer's parameter buffer; the last block
//                          signals "step done" to all peers.
// The summation order is the rank order on every rank, so all ranks hold identical bits and reruns repeat.
//
// Reference counterparts: ICollectives (src/Idrak.Abstraction/Cluster/Collectives.cs:34-80), the ring / naive
// algorithms and their device path (src/Idrak.Network/Collectives/Algorithms.cs:15-201,
// src/Idrak.Network/Abstractions/HostCollectives.cs:197-286), bucketed gradient reduction
// (src/Idrak.Network/Training/GradientReduction.cs:396-640) and ZeRO-style sharding (Sharding.cs:229-338).
// There the reduction runs on the CPU over host-staged buckets; here it runs inside the kernels above.
#include "comm.cuh"

namespace idrak {

// ---------------------------------------------------------------------------
// epoch / barrier helpers
// ---------------------------------------------------------------------------
__global__ void comm_bump_epoch_kernel(CommCtx c) {
  if (threadIdx.x == 0) *c.epoch = *c.epoch + 1;
}

// channel-wide barrier: publish the epoch, wait for everyone
__global__ void comm_barrier_kernel(CommCtx c, int channel) {
  const uint32_t e = *c.epoch;
  signal_peers(c, channel, e);
  wait_peers(c, channel, e, 20);
}

// wait only (used by tests to exercise the bounded wait with a flag nobody sets, and by the step-done fence)
__global__ void comm_wait_kernel(CommCtx c, int channel, uint32_t add) {
  wait_peers(c, channel, *c.epoch + add, 21);
}

// ---------------------------------------------------------------------------
// one-shot all-reduce of n <= slot_floats floats (sum or max), result identical on all ranks
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(CommCtx c, const float* __restrict__ in,
                                                                float* __restrict__ out, int n, int op_max,
                                                                int channel) {
  const uint32_t e = *c.epoch;
  // my values -> slot [rank] of every peer
  for (int i = threadIdx.x; i < n * c.world; i += blockDim.x) {
    const int p = i / n, k = i - p * n;
    c.slots[p][c.rank * c.slot_floats + k] = in[k];
  }
  __syncthreads();
  signal_peers(c, channel, e);
  if (!wait_peers(c, channel, e, 22)) return;
  for (int k = threadIdx.x; k < n; k += blockDim.x) {
    float acc = __ldcg(c.slots[c.rank] + k);
    for (int p = 1; p < c.world; ++p) {
      const float v = __ldcg(c.slots[c.rank] + p * c.slot_floats + k);
      acc = op_max ? fmaxf(acc, v) : acc + v;
    }
    out[k] = acc;
  }
  // second phase of the channel: nobody overwrites the slots before all ranks have read them
  __syncthreads();
  signal_peers(c, channel + 1, e);
  wait_peers(c, channel + 1, e, 23);
}

// ---------------------------------------------------------------------------
// reduce-scatter / all-gather / all-reduce / broadcast on symmetric buffers
//   bufs[p]   rank p's buffer (n elements); slices of n / world elements, slice r belongs to rank r
// ---------------------------------------------------------------------------
struct PeerPtrs {
  void* p[kMaxRanks];
};

// out (local, n/world elements, fp32 or bf16) = sum over ranks of slice `rank` of their buffers
template <bool kBf16>
__global__ void __launch_bounds__(512) reduce_scatter_kernel(CommCtx c, PeerPtrs bufs, void* __restrict__ out,
                                                             long long n_slice, int out_fp32, int channel,
                                                             float scale) {
  const uint32_t e = *c.epoch;
  if (blockIdx.x == 0) signal_peers(c, channel, e);   // my buffer is complete (stream order) -> tell everyone
  if (!wait_peers(c, channel, e, 24)) return;
  const long long base = (long long)c.rank * n_slice;
  constexpr int V = kBf16 ? 8 : 4;
  const long long nv = n_slice / V;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
      if (p < c.world) {
        if (kBf16) {
          uint4 v = ld_peer16(static_cast<const __nv_bfloat16*>(bufs.p[p]) + base + i * 8);
          accum_bf16x8(acc, v, 1.f);
        } else {
          float4 v = __ldcg(reinterpret_cast<const float4*>(static_cast<const float*>(bufs.p[p]) + base + i * 4));
          acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= scale;
    if (out_fp32) {
      float* o = static_cast<float*>(out) + i * V;
      *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (kBf16) *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out) + i * V;
      if (kBf16) {
        uint4 w;
        w.x = pack_bf16x2(acc[0], acc[1]); w.y = pack_bf16x2(acc[2], acc[3]);
        w.z = pack_bf16x2(acc[4], acc[5]); w.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(o) = w;
      } else {
        uint2 w;
        w.x = pack_bf16x2(acc[0], acc[1]); w.y = pack_bf16x2(acc[2], acc[3]);
        *reinterpret_cast<uint2*>(o) = w;
      }
    }
  }
  // the peers may not overwrite their buffers until everyone has read them
  if (last_block(c, channel)) {
    signal_peers(c, channel + 1, e);
    wait_peers(c, channel + 1, e, 29);   // when this kernel ends, every peer has finished reading my buffer
  }
}

// every rank's slice `rank` of `in` (local, slice_bytes) is stored into all peers' bufs; uses channel and channel + 1
__global__ void __launch_bounds__(512) all_gather_kernel(CommCtx c, PeerPtrs bufs, const void* __restrict__ in,
                                                         long long slice_bytes, int channel) {
  const uint32_t e = *c.epoch;
  // Nobody stores into a peer's buffer before that peer says it is done with the previous contents: a rank
  // publishes "my buffer is free" on channel + 1 when this kernel starts (stream order puts that after its last
  // consumer of the earlier result) and every block waits for all peers' word before its first store.
  if (blockIdx.x == 0) signal_peers(c, channel + 1, e);
  if (!wait_peers(c, channel + 1, e, 33)) return;
  const long long nv = slice_bytes / 16;
  const uint4* src = static_cast<const uint4*>(in);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
      if (p < c.world) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(bufs.p[p]) + (long long)c.rank * slice_bytes);
        dst[i] = v;
      }
    }
  }
  if (last_block(c, channel)) {
    signal_peers(c, channel, e);
    wait_peers(c, channel, e, 25);   // on return every peer's slice has landed in my buffer
  }
}

// two-shot all-reduce in place on symmetric buffers of n elements (n % (world * 8) == 0)
template <bool kBf16>
__global__ void __launch_bounds__(512) allreduce_twoshot_kernel(CommCtx c, PeerPtrs bufs, long long n_slice,
                                                                int channel, float scale) {
  const uint32_t e = *c.epoch;
  if (blockIdx.x == 0) signal_peers(c, channel, e);
  if (!wait_peers(c, channel, e, 26)) return;
  const long long base = (long long)c.rank * n_slice;
  constexpr int V = kBf16 ? 8 : 4;
  const long long nv = n_slice / V;
  // phase 1+2 fused per vector: reduce my slice from all peers, store the result into every peer (including me)
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    uint4 vals[kMaxRanks];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < c.world) vals[p] = ld_peer16(static_cast<const char*>(bufs.p[p]) + (base + i * V) * (kBf16 ? 2 : 4));
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
      if (p < c.world) {
        if (kBf16) accum_bf16x8(acc, vals[p], 1.f);
        else {
          acc[0] += __uint_as_float(vals[p].x); acc[1] += __uint_as_float(vals[p].y);
          acc[2] += __uint_as_float(vals[p].z); acc[3] += __uint_as_float(vals[p].w);
        }
      }
    }
    uint4 w;
    if (kBf16) {
      w.x = pack_bf16x2(acc[0] * scale, acc[1] * scale); w.y = pack_bf16x2(acc[2] * scale, acc[3] * scale);
      w.z = pack_bf16x2(acc[4] * scale, acc[5] * scale); w.w = pack_bf16x2(acc[6] * scale, acc[7] * scale);
    } else {
      w.x = __float_as_uint(acc[0] * scale); w.y = __float_as_uint(acc[1] * scale);
      w.z = __float_as_uint(acc[2] * scale); w.w = __float_as_uint(acc[3] * scale);
    }
    // Nobody else reads slice `rank` (only its owner reduces it), so it can be overwritten at once.
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < c.world)
        *reinterpret_cast<uint4*>(static_cast<char*>(bufs.p[p]) + (base + i * V) * (kBf16 ? 2 : 4)) = w;
  }
  if (last_block(c, channel)) {
    signal_peers(c, channel + 1, e);
    wait_peers(c, channel + 1, e, 27);
  }
}

// root's buffer -> everyone (root pushes)
__global__ void __launch_bounds__(512) broadcast_kernel(CommCtx c, PeerPtrs bufs, long long bytes, int root,
                                                        int channel) {
  const uint32_t e = *c.epoch;
  // receivers publish "my buffer is free" (channel + 1) in stream order after their last reader of the old contents;
  // the root stores nothing before it has every receiver's word
  if (c.rank != root && blockIdx.x == 0) signal_peers(c, channel + 1, e);
  if (c.rank == root) {
    if (!wait_peers(c, channel + 1, e, 34, root)) return;
    const long long nv = bytes / 16;
    const uint4* src = static_cast<const uint4*>(bufs.p[root]);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      const uint4 v = src[i];
#pragma unroll
      for (int p = 0; p < kMaxRanks; ++p)
        if (p < c.world && p != root) static_cast<uint4*>(bufs.p[p])[i] = v;
    }
    if (last_block(c, channel)) signal_peers(c, channel, e);
  } else if (blockIdx.x == 0) {
    // wait for the root only: thread `root` polls
    const uint32_t* f = c.flags[c.rank] + channel * kMaxRanks + root;
    if (threadIdx.x == 0) {
      uint64_t t0 = 0;
      uint32_t polls = 0;
      while (int32_t(ld_acquire_sys(f) - e) < 0) {
        if ((++polls & 63u) == 0u) {
          const uint64_t now = global_timer_ns();
          if (t0 == 0) t0 = now;
          if (now - t0 > IDRAK_WAIT_BUDGET_NS) {
            report(c.st, kTimeoutPeerFlag, (28u << 16) | (uint32_t(channel) << 4) | root, e);
            break;
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// fused data-parallel step
// ---------------------------------------------------------------------------
// Bucket b covers flat elements [start, start + len) with len % (world * 8) == 0; rank r owns the sub-slice
// [start + r*len/world, start + (r+1)*len/world). Its reduced fp32 gradient goes to shard_grad + shard_off.
struct DpBucket {
  long long start, len, shard_off;
};

// U vectors per thread and pass: all U * world 16-byte loads of a pass are issued before the first one is used, so a
// thread keeps about eight peer loads in flight whatever the world size (U = 4 / 2 / 1 for 2 / 4 / 8 ranks); with one
// load per rank and pass a two-rank group had a single NVLink read outstanding per thread and stayed latency-bound.
template <int U>
__global__ void __launch_bounds__(512) dp_reduce_scatter_kernel(CommCtx c, PeerPtrs grads, DpBucket bk,
                                                                float* __restrict__ shard_grad,
                                                                float* __restrict__ sumsq_partial,
                                                                const float* __restrict__ rank_weights,
                                                                int channel) {
  __shared__ float red[16];
  const uint32_t e = *c.epoch;
  if (blockIdx.x == 0) signal_peers(c, channel, e);      // my gradients of this bucket are complete
  if (!wait_peers(c, channel, e, 30)) return;
  float w[kMaxRanks];
#pragma unroll
  for (int p = 0; p < kMaxRanks; ++p) w[p] = (p < c.world) ? (rank_weights ? rank_weights[p] : 1.f / c.world) : 0.f;
  const long long slice = bk.len / c.world;
  const long long base = bk.start + (long long)c.rank * slice;
  const long long nv = slice / 8;
  float sq = 0.f;
  constexpr int kRanksHere = kMaxRanks / U;             // the launcher picks U so that world <= kMaxRanks / U
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nv; i0 += stride * U) {
    uint4 vals[U][kRanksHere];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
#pragma unroll
      for (int p = 0; p < kRanksHere; ++p)
        if (p < c.world && i < nv) vals[u][p] = ld_peer16(static_cast<const __nv_bfloat16*>(grads.p[p]) + base + i * 8);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nv) break;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int p = 0; p < kRanksHere; ++p)
        if (p < c.world) accum_bf16x8(acc, vals[u][p], w[p]);
      float* o = shard_grad + bk.shard_off + i * 8;
      *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
      for (int j = 0; j < 8; ++j) sq += acc[j] * acc[j];
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.f;
    for (int i = 0; i < int(blockDim.x >> 5); ++i) r += red[i];
    sumsq_partial[blockIdx.x] = r;
  }
}

// hyper block layout shared with adamw.cu
enum { kHLr = 0, kHBeta1, kHBeta2, kHEps, kHBc1, kHBc2, kHClipScale, kHGradNorm, kHMaxNorm, kHGradScale };

// One block. partials: [n_partials] sums of squares of this rank's shard gradient -> global norm -> clip scale.
__global__ void __launch_bounds__(256) dp_norm_exchange_kernel(CommCtx c, const float* __restrict__ partials,
                                                               int n_partials, float* __restrict__ hyper,
                                                               int channel) {
  __shared__ float red[8];
  const uint32_t e = *c.epoch;
  float s = 0.f;
  for (int i = threadIdx.x; i < n_partials; i += blockDim.x) s += partials[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < c.world) {
    float mine = 0.f;
    for (int i = 0; i < 8; ++i) mine += red[i];
    c.slots[threadIdx.x][c.rank * c.slot_floats + 0] = mine;
  }
  __syncthreads();
  signal_peers(c, channel, e);
  if (!wait_peers(c, channel, e, 31)) return;
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int p = 0; p < c.world; ++p) total += __ldcg(c.slots[c.rank] + p * c.slot_floats + 0);
    const float gs = hyper[kHGradScale];
    const float norm = sqrtf(total) * fabsf(gs);
    const float max_norm = hyper[kHMaxNorm];
    float scale = 1.f;
    if (max_norm > 0.f && norm > max_norm) scale = max_norm / (norm + 1e-6f);
    if (!isfinite(norm)) scale = 0.f;
    hyper[kHGradNorm] = norm;
    hyper[kHClipScale] = scale;
  }
  __syncthreads();
  signal_peers(c, channel + 1, e);      // slot may be reused once everyone has read it
  wait_peers(c, channel + 1, e, 32);
}

// AdamW over this rank's shard + all-gather of the new bf16 weights into every peer's parameter buffer.
// decay_flags: one byte per 128-element group of the flat buffer (1 = weight decay applies).
__global__ void __launch_bounds__(512) dp_adamw_allgather_kernel(CommCtx c, PeerPtrs params, DpBucket bk,
                                                                 const float* __restrict__ shard_grad,
                                                                 float* __restrict__ master, float* __restrict__ m,
                                                                 float* __restrict__ v,
                                                                 const uint8_t* __restrict__ decay_flags,
                                                                 const float* __restrict__ hyper, float weight_decay,
                                                                 int channel, int signal_done) {
  const float lr = hyper[kHLr], b1 = hyper[kHBeta1], b2 = hyper[kHBeta2], eps = hyper[kHEps];
  const float bc1 = hyper[kHBc1], bc2_sqrt = sqrtf(hyper[kHBc2]);
  const float gscale = hyper[kHClipScale] * hyper[kHGradScale];
  const float step_size = lr / bc1;
  const long long slice = bk.len / c.world;
  const long long base = bk.start + (long long)c.rank * slice;
  const long long nv = slice / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const long long so = bk.shard_off + i * 8;
    const long long flat = base + i * 8;
    const float decay = decay_flags[flat >> 7] ? (1.f - lr * weight_decay) : 1.f;
    float g[8], mm[8], vv[8], pp[8];
    *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(shard_grad + so);
    *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(shard_grad + so + 4);
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(m + so);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(m + so + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + so);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + so + 4);
    *reinterpret_cast<float4*>(pp) = *reinterpret_cast<const float4*>(master + so);
    *reinterpret_cast<float4*>(pp + 4) = *reinterpret_cast<const float4*>(master + so + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gscale;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      pp[j] = pp[j] * decay - step_size * mm[j] / (sqrtf(vv[j]) / bc2_sqrt + eps);
    }
    *reinterpret_cast<float4*>(m + so) = *reinterpret_cast<float4*>(mm);
    *reinterpret_cast<float4*>(m + so + 4) = *reinterpret_cast<float4*>(mm + 4);
    *reinterpret_cast<float4*>(v + so) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(v + so + 4) = *reinterpret_cast<float4*>(vv + 4);
    *reinterpret_cast<float4*>(master + so) = *reinterpret_cast<float4*>(pp);
    *reinterpret_cast<float4*>(master + so + 4) = *reinterpret_cast<float4*>(pp + 4);
    uint4 w;
    w.x = pack_bf16x2(pp[0], pp[1]); w.y = pack_bf16x2(pp[2], pp[3]);
    w.z = pack_bf16x2(pp[4], pp[5]); w.w = pack_bf16x2(pp[6], pp[7]);
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < c.world) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[p]) + flat) = w;
  }
  if (signal_done && last_block(c, channel)) signal_peers(c, channel, *c.epoch);
}

static inline int comm_grid(long long vectors, int threads, int max_blocks) {
  long long b = (vectors + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return int(b);
}

}  // namespace idrak

using namespace idrak;

// ---------------------------------------------------------------------------
// host: symmetric allocations and IPC
// ---------------------------------------------------------------------------
IDRAK_API int idrak_symm_alloc(void** out, long long bytes) {
  cudaError_t e = cudaMalloc(out, size_t(bytes));
  if (e != cudaSuccess) return int(e);
  e = cudaMemset(*out, 0, size_t(bytes));
  return int(e);
}
IDRAK_API int idrak_symm_free(void* p) { return int(cudaFree(p)); }
IDRAK_API int idrak_ipc_handle_bytes() { return int(sizeof(cudaIpcMemHandle_t)); }
IDRAK_API int idrak_ipc_get_handle(void* p, void* handle_out) {
  return int(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out), p));
}
IDRAK_API int idrak_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return int(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
IDRAK_API int idrak_ipc_close(void* p) { return int(cudaIpcCloseMemHandle(p)); }
IDRAK_API int idrak_comm_ctx_bytes() { return int(sizeof(CommCtx)); }
IDRAK_API int idrak_comm_max_ranks() { return kMaxRanks; }
IDRAK_API int idrak_comm_flag_channels() { return kFlagChannels; }
IDRAK_API long long idrak_comm_flag_bytes() { return (long long)kFlagChannels * kMaxRanks * 4; }

// Fill a CommCtx (host struct passed by value to the launchers below).
IDRAK_API void idrak_comm_ctx_init(void* ctx_out, int rank, int world, void* const* flag_ptrs,
                                   void* const* slot_ptrs, int slot_floats, void* epoch, void* counters) {
  CommCtx c;
  memset(&c, 0, sizeof(c));
  c.rank = rank;
  c.world = world;
  for (int p = 0; p < world && p < kMaxRanks; ++p) {
    c.flags[p] = static_cast<uint32_t*>(flag_ptrs[p]);
    c.slots[p] = static_cast<float*>(slot_ptrs[p]);
  }
  c.slot_floats = slot_floats;
  c.epoch = static_cast<uint32_t*>(epoch);
  c.counters = static_cast<uint32_t*>(counters);
  c.st = status_device_ptr();
  memcpy(ctx_out, &c, sizeof(c));
}

// A kernel signals on `channel` and, for its second phase, on the channel after it: both rows must lie inside the
// flag area of kFlagChannels rows that every rank allocated.
static inline bool bad_channel(int channel) { return channel < 0 || channel + 1 >= kFlagChannels; }

static inline CommCtx load_ctx(const void* ctx) {
  CommCtx c;
  memcpy(&c, ctx, sizeof(c));
  return c;
}
static inline PeerPtrs load_ptrs(void* const* ptrs, int world) {
  PeerPtrs p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < world && i < kMaxRanks; ++i) p.p[i] = ptrs[i];
  return p;
}

IDRAK_API int idrak_comm_bump_epoch(const void* ctx, void* stream_) {
  comm_bump_epoch_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(load_ctx(ctx));
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_comm_barrier(const void* ctx, int channel, void* stream_) {
  if (bad_channel(channel)) return -3;
  comm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(load_ctx(ctx), channel);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_comm_wait(const void* ctx, int channel, unsigned add, void* stream_) {
  if (bad_channel(channel)) return -3;
  comm_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(load_ctx(ctx), channel, add);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_allreduce_oneshot(const void* ctx, const float* in, float* out, int n, int op_max, int channel,
                                      void* stream_) {
  if (bad_channel(channel)) return -3;
  CommCtx c = load_ctx(ctx);
  if (n > c.slot_floats) return -2;
  allreduce_oneshot_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream_)>>>(c, in, out, n, op_max, channel);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_reduce_scatter(const void* ctx, void* const* bufs, void* out, long long n, int bf16,
                                   int out_fp32, float scale, int channel, int max_blocks, void* stream_) {
  if (bad_channel(channel)) return -3;
  CommCtx c = load_ctx(ctx);
  const int V = bf16 ? 8 : 4;
  if (n % (c.world * V)) return -2;
  const long long n_slice = n / c.world;
  PeerPtrs p = load_ptrs(bufs, c.world);
  const int grid = comm_grid(n_slice / V, 512, max_blocks > 0 ? max_blocks : 64);
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  if (bf16) reduce_scatter_kernel<true><<<grid, 512, 0, s>>>(c, p, out, n_slice, out_fp32, channel, scale);
  else reduce_scatter_kernel<false><<<grid, 512, 0, s>>>(c, p, out, n_slice, out_fp32, channel, scale);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_all_gather(const void* ctx, void* const* bufs, const void* in, long long slice_bytes,
                               int channel, int max_blocks, void* stream_) {
  if (bad_channel(channel)) return -3;
  CommCtx c = load_ctx(ctx);
  if (slice_bytes % 16) return -2;
  PeerPtrs p = load_ptrs(bufs, c.world);
  const int grid = comm_grid(slice_bytes / 16, 512, max_blocks > 0 ? max_blocks : 64);
  all_gather_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream_)>>>(c, p, in, slice_bytes, channel);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_allreduce_twoshot(const void* ctx, void* const* bufs, long long n, int bf16, float scale,
                                      int channel, int max_blocks, void* stream_) {
  if (bad_channel(channel)) return -3;
  CommCtx c = load_ctx(ctx);
  const int V = bf16 ? 8 : 4;
  if (n % (c.world * V)) return -2;
  PeerPtrs p = load_ptrs(bufs, c.world);
  const long long n_slice = n / c.world;
  const int grid = comm_grid(n_slice / V, 512, max_blocks > 0 ? max_blocks : 64);
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  if (bf16) allreduce_twoshot_kernel<true><<<grid, 512, 0, s>>>(c, p, n_slice, channel, scale);
  else allreduce_twoshot_kernel<false><<<grid, 512, 0, s>>>(c, p, n_slice, channel, scale);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_broadcast(const void* ctx, void* const* bufs, long long bytes, int root, int channel,
                              int max_blocks, void* stream_) {
  if (bad_channel(channel)) return -3;
  CommCtx c = load_ctx(ctx);
  if (bytes % 16) return -2;
  PeerPtrs p = load_ptrs(bufs, c.world);
  const int grid = comm_grid(bytes / 16, 512, max_blocks > 0 ? max_blocks : 64);
  broadcast_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream_)>>>(c, p, bytes, root, channel);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_dp_reduce_scatter(const void* ctx, void* const* grads, long long start, long long len,
                                      long long shard_off, float* shard_grad, float* sumsq_partial,
                                      const float* rank_weights, int channel, int blocks, void* stream_) {
  if (bad_channel(channel)) return -3;
  CommCtx c = load_ctx(ctx);
  if (len % (c.world * 8)) return -2;
  PeerPtrs p = load_ptrs(grads, c.world);
  DpBucket bk{start, len, shard_off};
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (c.world <= kMaxRanks / 4)
    dp_reduce_scatter_kernel<4><<<blocks, 512, 0, stream>>>(c, p, bk, shard_grad, sumsq_partial, rank_weights, channel);
  else if (c.world <= kMaxRanks / 2)
    dp_reduce_scatter_kernel<2><<<blocks, 512, 0, stream>>>(c, p, bk, shard_grad, sumsq_partial, rank_weights, channel);
  else
    dp_reduce_scatter_kernel<1><<<blocks, 512, 0, stream>>>(c, p, bk, shard_grad, sumsq_partial, rank_weights, channel);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_dp_norm_exchange(const void* ctx, const float* partials, int n_partials, float* hyper,
                                     int channel, void* stream_) {
  if (bad_channel(channel)) return -3;
  dp_norm_exchange_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream_)>>>(load_ctx(ctx), partials, n_partials,
                                                                            hyper, channel);
  note_launches(1);
  return int(cudaGetLastError());
}
IDRAK_API int idrak_dp_adamw_allgather(const void* ctx, void* const* params, long long start, long long len,
                                       long long shard_off, const float* shard_grad, float* master, float* m,
                                       float* v, const void* decay_flags, const float* hyper, float weight_decay,
                                       int channel, int signal_done, int blocks, void* stream_) {
  if (bad_channel(channel)) return -3;
  CommCtx c = load_ctx(ctx);
  if (len % (c.world * 8)) return -2;
  PeerPtrs p = load_ptrs(params, c.world);
  DpBucket bk{start, len, shard_off};
  dp_adamw_allgather_kernel<<<blocks, 512, 0, static_cast<cudaStream_t>(stream_)>>>(
      c, p, bk, shard_grad, master, m, v, static_cast<const uint8_t*>(decay_flags), hyper, weight_decay, channel,
      signal_done);
  note_launches(1);
  return int(cudaGetLastError());
}
