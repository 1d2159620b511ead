// Decode-time attention over a block-table ("paged") KV cache, and the kernel that writes new keys / values
// into it.
//
// Cache layout: k_cache, v_cache = [num_blocks, block_size, kv_heads, head_dim] bf16; a sequence's blocks are
// listed in block_table[seq, :]; token t of a sequence lives in block block_table[seq, t / block_size] at
// offset t % block_size.
//
// paged_decode_kernel: grid (sequences, kv heads, splits). One CTA serves the G = heads / kv_heads query heads
// that share a KV head over one contiguous share of the sequence's key blocks: each of its 4 warps stages
// 32-key tiles of K and V in shared memory with 128-bit coalesced loads, lane l scores key l against the G
// queries, the warp keeps an online softmax per query head, and lanes own slices of the head dimension for
// the P·V accumulation. Splits write (max, sum, partial output) and decode_merge_kernel combines them in split
// order. The kernel is bandwidth bound (each K / V byte is read once), which is why it runs on the FMA pipes.
//
// Reference counterparts: attention_decode_{f32,int8,bf16} (split over blocks, last block merges;
// src/Idrak.Gpu/Cuda/PtxKernels.Rows.cs:2047-2060), kv_write_{f32,bf16} (PtxKernels.Decoding.cs:12),
// KeyValuePages (src/Idrak.Abstraction/Generation/KeyValuePages.cs:20-34) whose pages the reference copies into a
// contiguous cache instead of attending over them in place.
#include "common.cuh"

namespace idrak {

constexpr int kDecWarps = 4;
constexpr int kDecTile = 32;       // keys per warp tile
constexpr int kDecMaxGroup = 16;   // query heads per KV head

struct DecodeParams {
  const __nv_bfloat16* q;        // [seqs, H, D]
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_table;        // [seqs, max_blocks]
  const int* seq_lens;           // [seqs]
  __nv_bfloat16* out;            // [seqs, H, D]
  float* partial;                // [seqs, H, splits, D + 2]
  int H, Hkv, D, block_size, max_blocks, splits;
  float scale_log2;
  int window;                    // 0 = full; else attend to the last `window` positions only
};

template <int D>
__global__ void __launch_bounds__(kDecWarps * 32) paged_decode_kernel(const DecodeParams p) {
  constexpr int kRow = D * 2 + 16;                       // padded shared-memory row (bytes)
  constexpr int DPL = D / 32;                            // head-dim elements per lane in the P·V phase
  extern __shared__ uint8_t dsm[];
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* sq = reinterpret_cast<float*>(dsm);                                  // [G][D] queries, pre-scaled
  uint8_t* sk = dsm + kDecMaxGroup * D * 4 + warp * (2 * kDecTile * kRow);     // this warp's K tile
  uint8_t* sv = sk + kDecTile * kRow;                                          // and V tile
  float* smerge = reinterpret_cast<float*>(dsm + kDecMaxGroup * D * 4 + kDecWarps * 2 * kDecTile * kRow);

  const int len = p.seq_lens[seq];
  const int first_pos = (p.window > 0 && len > p.window) ? len - p.window : 0;
  // this split's range of key tiles
  const int tiles = (len + kDecTile - 1) / kDecTile;
  const int first_tile = first_pos / kDecTile;
  const int span = tiles - first_tile;
  const int per = (span + p.splits - 1) / p.splits;
  const int t0 = first_tile + split * per, t1 = min(tiles, t0 + per);

  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    sq[i] = __bfloat162float(p.q[(size_t(seq) * p.H + kvh * G + g) * D + d]) * p.scale_log2;
  }
  __syncthreads();

  float m[kDecMaxGroup], l[kDecMaxGroup], acc[kDecMaxGroup][DPL];
#pragma unroll
  for (int g = 0; g < kDecMaxGroup; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[g][j] = 0.f;
  }
  const size_t tok_stride = size_t(p.Hkv) * D;            // elements between tokens of a block
  const int* table = p.block_table + size_t(seq) * p.max_blocks;

  for (int t = t0 + warp; t < t1; t += kDecWarps) {
    const int key0 = t * kDecTile;
    // ---- stage 32 keys x D of K and V: chunk c of key r <- 16 bytes
    constexpr int kChunks = D / 8;
    for (int i = lane; i < kDecTile * kChunks; i += 32) {
      const int r = i / kChunks, c = i - r * kChunks;
      const int pos = key0 + r;
      uint4 kv4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
      if (pos < len) {
        const int blk = table[pos / p.block_size];
        const size_t off = (size_t(blk) * p.block_size + pos % p.block_size) * tok_stride + size_t(kvh) * D + c * 8;
        kv4 = *reinterpret_cast<const uint4*>(p.k_cache + off);
        vv4 = *reinterpret_cast<const uint4*>(p.v_cache + off);
      }
      *reinterpret_cast<uint4*>(sk + r * kRow + c * 16) = kv4;
      *reinterpret_cast<uint4*>(sv + r * kRow + c * 16) = vv4;
    }
    __syncwarp();
    // ---- scores: lane = key
    const int pos = key0 + lane;
    const bool valid = pos < len && pos >= first_pos;
    float s[kDecMaxGroup];
#pragma unroll
    for (int g = 0; g < kDecMaxGroup; ++g) s[g] = 0.f;
    for (int c = 0; c < kChunks; ++c) {
      const uint4 kk = *reinterpret_cast<const uint4*>(sk + lane * kRow + c * 16);
      float kf[8];
      float2 f;
      f = unpack_bf16x2(kk.x); kf[0] = f.x; kf[1] = f.y;
      f = unpack_bf16x2(kk.y); kf[2] = f.x; kf[3] = f.y;
      f = unpack_bf16x2(kk.z); kf[4] = f.x; kf[5] = f.y;
      f = unpack_bf16x2(kk.w); kf[6] = f.x; kf[7] = f.y;
#pragma unroll
      for (int g = 0; g < kDecMaxGroup; ++g) {
        if (g < G) {
          const float* qg = sq + g * D + c * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) s[g] += qg[j] * kf[j];
        }
      }
    }
    // ---- online softmax per query head, then P·V with lanes owning head-dim slices
#pragma unroll
    for (int g = 0; g < kDecMaxGroup; ++g) {
      if (g < G) {
        const float sc = valid ? s[g] : -INFINITY;
        const float mt = warp_max(sc);
        const float mn = fmaxf(m[g], mt);
        const float alpha = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
        const float pr = (valid && mn != -INFINITY) ? exp2f(sc - mn) : 0.f;
        l[g] = l[g] * alpha + warp_sum(pr);
        m[g] = mn;
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[g][j] *= alpha;
        for (int r = 0; r < kDecTile; ++r) {
          const float pw = __shfl_sync(0xffffffffu, pr, r);
          if (pw != 0.f) {
            const __nv_bfloat16* vr = reinterpret_cast<const __nv_bfloat16*>(sv + r * kRow) + lane * DPL;
#pragma unroll
            for (int j = 0; j < DPL; ++j) acc[g][j] += pw * __bfloat162float(vr[j]);
          }
        }
      }
    }
    __syncwarp();
  }

  // ---- combine the 4 warps of the CTA (in warp order), then write the split's partial or the final output
  // smerge layout: [warp][g][D + 2]
#pragma unroll
  for (int g = 0; g < kDecMaxGroup; ++g) {
    if (g < G) {
      float* dst = smerge + (size_t(warp) * kDecMaxGroup + g) * (D + 2);
#pragma unroll
      for (int j = 0; j < DPL; ++j) dst[lane * DPL + j] = acc[g][j];
      if (lane == 0) { dst[D] = m[g]; dst[D + 1] = l[g]; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, smerge[(size_t(w) * kDecMaxGroup + g) * (D + 2) + D]);
    float ll = 0.f, oo = 0.f;
    for (int w = 0; w < kDecWarps; ++w) {
      const float* src = smerge + (size_t(w) * kDecMaxGroup + g) * (D + 2);
      const float a = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - mm);
      ll += src[D + 1] * a;
      oo += src[d] * a;
    }
    const int head = kvh * G + g;
    if (p.splits == 1) {
      p.out[(size_t(seq) * p.H + head) * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
    } else {
      float* pp = p.partial + ((size_t(seq) * p.H + head) * p.splits + split) * (D + 2);
      pp[d] = oo;
      if (d == 0) { pp[D] = mm; pp[D + 1] = ll; }
    }
  }
}

// out[seq, head, :] = merge of the splits' partials, in split order
__global__ void decode_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int rows,
                                    int splits, int D) {
  const int row = blockIdx.x;
  if (row >= rows) return;
  const float* base = partial + size_t(row) * splits * (D + 2);
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, base[s * (D + 2) + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float ll = 0.f, oo = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* src = base + s * (D + 2);
      const float a = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - mm);
      ll += src[D + 1] * a;
      oo += src[d] * a;
    }
    out[size_t(row) * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
  }
}

// k / v rows of new tokens -> their cache slots. src rows hold heads packed [Hkv, D]; slot = block * block_size + offset.
__global__ void kv_write_paged_kernel(const __nv_bfloat16* __restrict__ k_src, const __nv_bfloat16* __restrict__ v_src,
                                      long long src_stride, const int* __restrict__ slots,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      int tokens, int row_elems) {
  const int chunks = row_elems / 8;
  const long long total = (long long)tokens * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / chunks), c = int(i - (long long)t * chunks);
    const int slot = slots[t];
    if (slot < 0) continue;     // padding token
    const uint4 kk = *reinterpret_cast<const uint4*>(k_src + t * src_stride + c * 8);
    const uint4 vv = *reinterpret_cast<const uint4*>(v_src + t * src_stride + c * 8);
    *reinterpret_cast<uint4*>(k_cache + size_t(slot) * row_elems + c * 8) = kk;
    *reinterpret_cast<uint4*>(v_cache + size_t(slot) * row_elems + c * 8) = vv;
  }
}

template <int D>
static size_t decode_smem() {
  return size_t(kDecMaxGroup) * D * 4 + size_t(kDecWarps) * 2 * kDecTile * (D * 2 + 16) +
         size_t(kDecWarps) * kDecMaxGroup * (D + 2) * 4;
}

}  // namespace idrak

using namespace idrak;

IDRAK_API long long idrak_decode_partial_floats(int seqs, int H, int D, int splits) {
  return splits > 1 ? (long long)seqs * H * splits * (D + 2) : 0;
}

IDRAK_API int idrak_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                 const int* seq_lens, void* out, float* partial, int seqs, int H, int Hkv, int D,
                                 int block_size, int max_blocks, int splits, float scale, int window, void* stream_) {
  if (D != 64 && D != 128) return -2;
  if (H % Hkv || H / Hkv > kDecMaxGroup) return -3;
  if (splits > 1 && !partial) return -4;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.partial = partial;
  p.H = H; p.Hkv = Hkv; p.D = D; p.block_size = block_size; p.max_blocks = max_blocks;
  p.splits = splits < 1 ? 1 : splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  dim3 grid(seqs, Hkv, p.splits);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(paged_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(decode_smem<64>()));
    cudaFuncSetAttribute(paged_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(decode_smem<128>()));
    configured = true;
  }
  if (D == 64) paged_decode_kernel<64><<<grid, kDecWarps * 32, decode_smem<64>(), s>>>(p);
  else paged_decode_kernel<128><<<grid, kDecWarps * 32, decode_smem<128>(), s>>>(p);
  note_launches(1);
  int rc = int(cudaGetLastError());
  if (rc) return rc;
  if (p.splits > 1) {
    decode_merge_kernel<<<seqs * H, D < 128 ? 64 : 128, 0, s>>>(partial, p.out, seqs * H, p.splits, D);
    note_launches(1);
    rc = int(cudaGetLastError());
  }
  return rc;
}

IDRAK_API int idrak_kv_write_paged(const void* k_src, const void* v_src, long long src_stride, const int* slots,
                                   void* k_cache, void* v_cache, int tokens, int row_elems, void* stream_) {
  if (row_elems % 8) return -2;
  const long long total = (long long)tokens * (row_elems / 8);
  long long want = (total + 255) / 256, cap = (long long)sm_count() * 8;
  kv_write_paged_kernel<<<int(want < 1 ? 1 : (want < cap ? want : cap)), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const __nv_bfloat16*>(k_src), static_cast<const __nv_bfloat16*>(v_src), src_stride, slots,
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), tokens, row_elems);
  note_launches(1);
  return int(cudaGetLastError());
}
