// Mixture-of-experts routing on the device: nothing here needs a host read, so a routed layer records into a CUDA graph.
//
//   route_choose   router logits [T, E] -> softmax, top-k expert ids (ties: lowest id) and their weights
//   route_count    how many of the T * k assignments each block of 1024 sends to each expert
//   route_offsets  one block: per-expert segment starts (each segment padded to a multiple of 128 rows so that no
//                  GEMM tile straddles two experts), per-(block, expert) bases, the expert of every 128-row tile, the
//                  number of tiles in use and the per-expert row ranges in units of 64 rows (the K blocks of the
//                  weight-gradient product)
//   route_place    destination row of every assignment: stable (assignments keep token order inside an expert), so the
//                  result is the same on every run
//   route_gather   permuted activations: dst row <- source token row (times a weight, for the backward pass); padding
//                  rows are written as zeros
//   route_combine  out[t] = sum_k w[t, k] * y[dst(t, k)] (+ residual); optionally dw[t, k] = <g[t], y[dst(t, k)]>
//
// The expert products themselves are the grouped modes of the dense tcgen05 GEMM (gemm_tcgen05.cu).
//
// Reference counterparts: route_choose / route_counts / route_offsets / route_place / expert_gated / expert_matmul
// (src/Idrak.Gpu/Cuda/PtxKernels.Routing.cs:12-35), MixtureOfExperts (src/Idrak/Layers/MixtureOfExperts.cs:34).
#include "common.cuh"

namespace idrak {

constexpr int kRouteBlock = 1024;      // assignments per block of the counting / placing kernels
constexpr int kRouteMaxExperts = 256;
constexpr int kRouteTile = 128;        // rows per GEMM tile: segments are padded to this

// One warp per token. E <= 256: lane l holds experts l, l + 32, ...
__global__ void __launch_bounds__(256) route_choose_kernel(const float* __restrict__ logits, int T, int E, int k,
                                                           int normalize, int* __restrict__ top_i,
                                                           float* __restrict__ top_w, float* __restrict__ probs) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  float v[kRouteMaxExperts / 32];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kRouteMaxExperts / 32; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? logits[size_t(t) * E + e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < kRouteMaxExperts / 32; ++j) {
    v[j] = (lane + 32 * j < E) ? __expf(v[j] - mx) : 0.f;
    sum += v[j];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int j = 0; j < kRouteMaxExperts / 32; ++j) {
    v[j] *= inv;
    if (probs && lane + 32 * j < E) probs[size_t(t) * E + lane + 32 * j] = v[j];
  }
  float picked_sum = 0.f;
  float my_w = 0.f;       // lane s keeps the weight of pick s
  int my_i = 0;
  for (int s = 0; s < k; ++s) {
    // largest remaining probability; among equals the lowest expert id
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kRouteMaxExperts / 32; ++j) {
      const int e = lane + 32 * j;
      if (e < E && (v[j] > best)) { best = v[j]; best_e = e; }      // ascending e per lane: first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
#pragma unroll
    for (int j = 0; j < kRouteMaxExperts / 32; ++j)
      if (lane + 32 * j == best_e) v[j] = -2.f;                     // taken
    picked_sum += best;
    if (lane == s) { my_w = best; my_i = best_e; }
  }
  if (lane < k) {
    top_i[size_t(t) * k + lane] = my_i;
    top_w[size_t(t) * k + lane] = normalize ? my_w / picked_sum : my_w;
  }
}

__global__ void __launch_bounds__(kRouteBlock) route_count_kernel(const int* __restrict__ top_i, int A, int E,
                                                                  int* __restrict__ block_hist) {
  __shared__ int hist[kRouteMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int a = blockIdx.x * kRouteBlock + threadIdx.x;
  if (a < A) atomicAdd(&hist[top_i[a]], 1);        // integer counts: the order of the additions does not matter
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[size_t(blockIdx.x) * E + e] = hist[e];
}

// One block of 256 threads; thread e (e < E) walks its expert's column of the block histogram.
// meta: [0] tiles in use, [1] rows in use (padded), [2 ...] reserved.
__global__ void __launch_bounds__(256) route_offsets_kernel(int* __restrict__ block_hist, int blocks, int E, int cap_tiles,
                                                            int* __restrict__ seg_start, int* __restrict__ seg_count,
                                                            int* __restrict__ tile_group, int* __restrict__ group_kb,
                                                            int* __restrict__ meta) {
  __shared__ int total[kRouteMaxExperts];
  __shared__ int start[kRouteMaxExperts + 1];
  const int e = threadIdx.x;
  if (e < E) {
    int run = 0;
    for (int b = 0; b < blocks; ++b) {
      const int c = block_hist[size_t(b) * E + e];
      block_hist[size_t(b) * E + e] = run;           // becomes the base of block b inside the expert's segment
      run += c;
    }
    total[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int x = 0; x < E; ++x) {
      start[x] = at;
      at += (total[x] + kRouteTile - 1) / kRouteTile * kRouteTile;
    }
    start[E] = at;
    meta[0] = at / kRouteTile;
    meta[1] = at;
  }
  __syncthreads();
  if (e < E) {
    seg_start[e] = start[e];
    seg_count[e] = total[e];
    group_kb[e] = start[e] / 64;
    for (int tile = start[e] / kRouteTile; tile < start[e + 1] / kRouteTile; ++tile) tile_group[tile] = e;
  }
  if (e == 0) group_kb[E] = start[E] / 64;
  for (int tile = start[E] / kRouteTile + threadIdx.x; tile < cap_tiles; tile += blockDim.x) tile_group[tile] = -1;
}

// Stable rank inside the block: assignment a is preceded by the assignments of the same expert in earlier warps of the
// block plus those in lower lanes of its own warp.
__global__ void __launch_bounds__(kRouteBlock) route_place_kernel(const int* __restrict__ top_i, int A, int E,
                                                                  const int* __restrict__ block_base,
                                                                  const int* __restrict__ seg_start,
                                                                  int* __restrict__ dst_of, int* __restrict__ row_of) {
  __shared__ int warp_hist[kRouteBlock / 32][kRouteMaxExperts];     // 32 KB
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (kRouteBlock / 32) * kRouteMaxExperts; i += blockDim.x)
    (&warp_hist[0][0])[i] = 0;
  __syncthreads();
  const int a = blockIdx.x * kRouteBlock + threadIdx.x;
  const bool live = a < A;
  const int e = live ? top_i[a] : -1;
  const unsigned same = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
  if (live && rank_in_warp == 0) warp_hist[warp][e] = __popc(same);
  __syncthreads();
  if (live) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_hist[w][e];
    const int dst = seg_start[e] + block_base[size_t(blockIdx.x) * E + e] + before + rank_in_warp;
    dst_of[a] = dst;
    row_of[dst] = a;
  }
}

// One warp per destination row; C % 8 == 0. row_of[dst] = assignment index (token = index / k) or -1 for padding.
__global__ void __launch_bounds__(256) route_gather_kernel(const __nv_bfloat16* __restrict__ src, long long src_ld,
                                                           const int* __restrict__ row_of, const float* __restrict__ w,
                                                           const int* __restrict__ meta, int k, int C,
                                                           __nv_bfloat16* __restrict__ out) {
  const int dst = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (dst >= meta[1]) return;
  const int lane = threadIdx.x & 31;
  const int a = row_of[dst];
  uint4* orow = reinterpret_cast<uint4*>(out + size_t(dst) * C);
  if (a < 0) {
    for (int c = lane; c < C / 8; c += 32) orow[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* srow = reinterpret_cast<const uint4*>(src + size_t(a / k) * src_ld);
  if (!w) {
    for (int c = lane; c < C / 8; c += 32) orow[c] = __ldg(srow + c);
    return;
  }
  const float f = w[a];
  for (int c = lane; c < C / 8; c += 32) {
    uint4 v = __ldg(srow + c);
    float2 p0 = unpack_bf16x2(v.x), p1 = unpack_bf16x2(v.y), p2 = unpack_bf16x2(v.z), p3 = unpack_bf16x2(v.w);
    v.x = pack_bf16x2(p0.x * f, p0.y * f);
    v.y = pack_bf16x2(p1.x * f, p1.y * f);
    v.z = pack_bf16x2(p2.x * f, p2.y * f);
    v.w = pack_bf16x2(p3.x * f, p3.y * f);
    orow[c] = v;
  }
}

// One warp per token: out[t] = sum_k w[t,k] * y[dst_of[t,k]] (+ residual[t]); with `g`, also dw[t,k] = <g[t], y[dst]>.
__global__ void __launch_bounds__(256) route_combine_kernel(const __nv_bfloat16* __restrict__ y,
                                                            const int* __restrict__ dst_of, const float* __restrict__ w,
                                                            const __nv_bfloat16* __restrict__ residual,
                                                            const __nv_bfloat16* __restrict__ g, float* __restrict__ dw,
                                                            int T, int k, int C, __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  if (out) {
    for (int c = lane; c < C / 8; c += 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int s = 0; s < k; ++s) {
        const float f = w ? w[size_t(t) * k + s] : 1.f;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + size_t(dst_of[size_t(t) * k + s]) * C) + c);
        float2 p;
        p = unpack_bf16x2(v.x); acc[0] += f * p.x; acc[1] += f * p.y;
        p = unpack_bf16x2(v.y); acc[2] += f * p.x; acc[3] += f * p.y;
        p = unpack_bf16x2(v.z); acc[4] += f * p.x; acc[5] += f * p.y;
        p = unpack_bf16x2(v.w); acc[6] += f * p.x; acc[7] += f * p.y;
      }
      if (residual) {
        const uint4 r = __ldg(reinterpret_cast<const uint4*>(residual + size_t(t) * C) + c);
        float2 p;
        p = unpack_bf16x2(r.x); acc[0] += p.x; acc[1] += p.y;
        p = unpack_bf16x2(r.y); acc[2] += p.x; acc[3] += p.y;
        p = unpack_bf16x2(r.z); acc[4] += p.x; acc[5] += p.y;
        p = unpack_bf16x2(r.w); acc[6] += p.x; acc[7] += p.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + size_t(t) * C)[c] = o;
    }
  }
  if (g && dw) {
    for (int s = 0; s < k; ++s) {
      const __nv_bfloat16* yr = y + size_t(dst_of[size_t(t) * k + s]) * C;
      float dot = 0.f;
      for (int c = lane; c < C / 8; c += 32) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(g + size_t(t) * C) + c);
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(yr) + c);
        float2 p, q;
        p = unpack_bf16x2(a.x); q = unpack_bf16x2(b.x); dot += p.x * q.x + p.y * q.y;
        p = unpack_bf16x2(a.y); q = unpack_bf16x2(b.y); dot += p.x * q.x + p.y * q.y;
        p = unpack_bf16x2(a.z); q = unpack_bf16x2(b.z); dot += p.x * q.x + p.y * q.y;
        p = unpack_bf16x2(a.w); q = unpack_bf16x2(b.w); dot += p.x * q.x + p.y * q.y;
      }
      dot = warp_sum(dot);
      if (lane == 0) dw[size_t(t) * k + s] = dot;
    }
  }
}

}  // namespace idrak

using namespace idrak;

// Rows the permuted buffers must hold for T tokens, k picks each, E experts: every segment may need up to 127 padding rows.
IDRAK_API int idrak_route_capacity(int T, int k, int E) {
  const long long rows = (long long)T * k + (long long)E * (kRouteTile - 1);
  return int((rows + kRouteTile - 1) / kRouteTile * kRouteTile);
}

// Sizes (ints) of the plan arrays for A = T * k assignments: block_hist blocks * E, seg_start E, seg_count E,
// tile_group cap / 128, group_kb E + 1, meta 4, dst_of A, row_of cap.
IDRAK_API int idrak_route_blocks(int A) { return (A + kRouteBlock - 1) / kRouteBlock; }

IDRAK_API int idrak_route_choose(const float* logits, int T, int E, int k, int normalize, int* top_i, float* top_w,
                                 float* probs, void* stream_) {
  if (E < 1 || E > kRouteMaxExperts || k < 1 || k > 32 || k > E) return -2;
  if (T <= 0) return 0;
  route_choose_kernel<<<(T + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream_)>>>(logits, T, E, k, normalize, top_i,
                                                                                  top_w, probs);
  note_launches(1);
  return int(cudaGetLastError());
}

// Builds the whole plan from top_i [A]: three launches and one memset, no host read.
IDRAK_API int idrak_route_plan(const int* top_i, int A, int E, int cap, int* block_hist, int* seg_start, int* seg_count,
                               int* tile_group, int* group_kb, int* meta, int* dst_of, int* row_of, void* stream_) {
  if (E < 1 || E > kRouteMaxExperts || A <= 0 || cap % kRouteTile) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int blocks = (A + kRouteBlock - 1) / kRouteBlock;
  int rc = int(cudaMemsetAsync(row_of, 0xff, size_t(cap) * sizeof(int), s));     // -1: padding
  if (rc) return rc;
  route_count_kernel<<<blocks, kRouteBlock, 0, s>>>(top_i, A, E, block_hist);
  route_offsets_kernel<<<1, 256, 0, s>>>(block_hist, blocks, E, cap / kRouteTile, seg_start, seg_count, tile_group,
                                         group_kb, meta);
  route_place_kernel<<<blocks, kRouteBlock, 0, s>>>(top_i, A, E, block_hist, seg_start, dst_of, row_of);
  note_launches(3);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_route_gather(const void* src, long long src_ld, const int* row_of, const float* w, const int* meta,
                                 int k, int C, int cap, void* out, void* stream_) {
  if (C % 8 || (src_ld % 8)) return -2;
  route_gather_kernel<<<(cap + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const __nv_bfloat16*>(src), src_ld, row_of, w, meta, k, C, static_cast<__nv_bfloat16*>(out));
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_route_combine(const void* y, const int* dst_of, const float* w, const void* residual, const void* g,
                                  float* dw, int T, int k, int C, void* out, void* stream_) {
  if (C % 8) return -2;
  if (T <= 0) return 0;
  route_combine_kernel<<<(T + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const __nv_bfloat16*>(y), dst_of, w, static_cast<const __nv_bfloat16*>(residual),
      static_cast<const __nv_bfloat16*>(g), dw, T, k, C, static_cast<__nv_bfloat16*>(out));
  note_launches(1);
  return int(cudaGetLastError());
}
