// Decode-time attention over a block-table ("paged") KV cache, and the kernel that writes new keys / values
// into it.
//
// Cache layout: k_cache, v_cache = [num_blocks, block_size, kv_heads, head_dim] bf16; a sequence's blocks are
// listed in block_table[seq, :]; token t of a sequence lives in block block_table[seq, t / block_size] at
// offset t % block_size.
//
// paged_decode_kernel: grid (sequences, kv heads, splits). One CTA serves the G = heads / kv_heads query heads
// that share a KV head over one contiguous share of the sequence's key blocks: each of its 4 warps stages
// 32-key tiles of K and V in shared memory with asynchronous 16-byte copies and runs Q·K^T and P·V as
// m16n8k16 tensor-core MMAs with the G query heads as the (padded) 16 rows, keeping an online softmax per row
// in registers. Splits write (max, sum, partial output) and decode_merge_kernel combines them in split
// order. The kernel is bound by the bytes of K and V (each is read once); warp-level MMAs are enough to keep up
// with them - a 16-row tile cannot feed tcgen05's 128-row instruction - while the FMA pipes are not.
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
  const __nv_bfloat16* q;        // [seqs, H, D], sequences q_stride elements apart
  long long q_stride;
  const __nv_bfloat16* k_cache;  // bf16 cache; with an int8 cache these point at int8 codes [blocks, block_size, Hkv, D]
  const __nv_bfloat16* v_cache;
  const float* k_scale;          // int8 cache: one scale per (slot, kv head), [blocks * block_size, Hkv]
  const float* v_scale;
  const int* block_table;        // [seqs, max_blocks]
  const int* seq_lens;           // [seqs]
  __nv_bfloat16* out;            // [seqs, H, D]
  float* partial;                // [seqs, H, splits, D + 2]
  int H, Hkv, D, block_size, max_blocks, splits;
  float scale_log2;
  int window;                    // 0 = full; else attend to the last `window` positions only
};

// ---- warp-level tensor-core pieces (mma.sync m16n8k16, bf16 in, fp32 accumulate). Decode attention is bound by
// the bytes of K and V; the tensor pipe only has to keep up with them, which these 16-row MMAs do with the G <= 16
// query heads of a KV head as the rows - the FMA pipes cannot (2 multiply-adds per cache byte).
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
// 16-byte asynchronous copy global -> shared; `bytes` = 0 writes zeros instead (keys past the sequence's end)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// wait until at most one of this thread's committed groups is still in flight (groups complete in order)
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// 16 int8 codes times a scale -> 16 bf16 values (two 16-byte words)
__device__ __forceinline__ void dequant16(const uint4& raw, float scale, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = float(int8_t(w[i] & 0xff)) * scale, b = float(int8_t((w[i] >> 8) & 0xff)) * scale;
    const float c = float(int8_t((w[i] >> 16) & 0xff)) * scale, d = float(int8_t(w[i] >> 24)) * scale;
    o[2 * i] = pack_bf16x2(a, b);
    o[2 * i + 1] = pack_bf16x2(c, d);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// KV8 = 1: the cache holds int8 codes with one scale per (slot, kv head) (norm_rope_kv's int8 mode). A tile's codes
// are staged into the upper half of each shared-memory row and expanded to bf16 in place - lane r owns row r and
// walks it front to back, and the bf16 written for chunk c never reaches the codes of a chunk not yet read - so the
// tensor-core part below is unchanged and the cache costs half the bytes.
template <int D, int KV8>
__global__ void __launch_bounds__(kDecWarps * 32) paged_decode_kernel(const DecodeParams p) {
  pdl_launch_dependents();     // a dependent launched programmatically may set itself up while this kernel runs
  constexpr int kRow = D * 2 + 16;                       // padded shared-memory row (bytes): conflict-free ldmatrix
  constexpr int kChunks = D / 8;                         // 16-byte chunks per key row
  constexpr int KS = D / 16;                             // k-steps of Q·K^T
  constexpr int NT = D / 8;                              // n-tiles of P·V
  extern __shared__ uint8_t dsm[];
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* sqb = dsm;                                                          // [16][kRow] queries (bf16), rows >= G zero
  uint8_t* sk = dsm + 16 * kRow + warp * (2 * kDecTile * kRow);                // this warp's K tile
  uint8_t* sv = sk + kDecTile * kRow;                                          // and V tile
  // the warps' partial outputs are merged in the space of the K / V tiles once every warp is done with them: the kernel
  // then needs 74 KB instead of 107 KB (head size 128) and three CTAs share an SM instead of two
  float* smerge = reinterpret_cast<float*>(dsm + 16 * kRow);

  const int len = p.seq_lens[seq];
  const int first_pos = (p.window > 0 && len > p.window) ? len - p.window : 0;
  const int tiles = (len + kDecTile - 1) / kDecTile;
  const int first_tile = first_pos / kDecTile;
  const int span = tiles - first_tile;
  const int per = (span + p.splits - 1) / p.splits;
  const int t0 = first_tile + split * per, t1 = min(tiles, t0 + per);

  // queries of the G heads of this KV head -> shared (bf16, rows padded to 16 with zeros)
  for (int i = threadIdx.x; i < 16 * kChunks; i += blockDim.x) {
    const int g = i / kChunks, c = i - g * kChunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (g < G) v = *reinterpret_cast<const uint4*>(p.q + size_t(seq) * p.q_stride + size_t(kvh * G + g) * D + c * 8);
    *reinterpret_cast<uint4*>(sqb + g * kRow + c * 16) = v;
  }
  __syncthreads();
  // A fragments of Q for every k-step: ldmatrix.x4 gives (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15),
  // (rows 8-15, k 8-15) = a0..a3
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldmatrix_x4(qa[ks], sqb + (lane & 15) * kRow + ks * 32 + (lane >> 4) * 16);

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows lane / 4 and lane / 4 + 8
  const size_t tok_stride = size_t(p.Hkv) * D;
  const int* table = p.block_table + size_t(seq) * p.max_blocks;

  // lane r looks up the cache slot of key row r of a tile once (one division and one table read per lane and tile);
  // the copy loops fetch a row's slot by shuffle, so a 16-byte copy costs a shuffle and a multiply-add, not a
  // division, a remainder and a table read
  auto slot_of = [&](int tile) {
    const int pos = tile * kDecTile + lane;
    return (tile < t1 && pos < len) ? table[pos / p.block_size] * p.block_size + pos % p.block_size : -1;
  };
  // one 32-key tile of K or V (bf16 cache) into a warp's buffer, one commit group
  auto copy_rows = [&](uint8_t* dst, const __nv_bfloat16* cache, int slots) {
#pragma unroll 4
    for (int i = lane; i < kDecTile * kChunks; i += 32) {
      const int r = i / kChunks, c = i - r * kChunks;                // kChunks is a power of two: shifts
      const int slot = __shfl_sync(0xffffffffu, slots, r);
      const bool live = slot >= 0;
      const size_t off = live ? size_t(slot) * tok_stride + size_t(kvh) * D + c * 8 : 0;
      cp_async16(dst + r * kRow + c * 16, cache + off, live ? 16 : 0);
    }
    cp_async_commit();
  };
  // bf16 cache: the copies run one step ahead of the arithmetic inside the warp's single pair of buffers - the keys of
  // the next tile are requested as soon as Q K^T of this tile has read its keys (they fly during the softmax and P V),
  // the values of the next tile once P V has read its values (they fly during the next Q K^T and softmax)
  // int8 cache: the same, with the codes of a tile staged in the upper half of each row and expanded in place by the
  // lane that owns the row once they have landed
  constexpr int kByteChunks = D / 16;                    // 16-byte chunks of int8 codes per key row
  auto copy_codes = [&](uint8_t* dst, const __nv_bfloat16* cache, int slots) {
    const int8_t* codes = reinterpret_cast<const int8_t*>(cache);
#pragma unroll 4
    for (int i = lane; i < kDecTile * kByteChunks; i += 32) {
      const int r = i / kByteChunks, c = i - r * kByteChunks;
      const int slot = __shfl_sync(0xffffffffu, slots, r);
      const bool live = slot >= 0;
      const size_t off = live ? size_t(slot) * tok_stride + size_t(kvh) * D + c * 16 : 0;
      cp_async16(dst + r * kRow + D + c * 16, codes + off, live ? 16 : 0);
    }
    cp_async_commit();
  };
  auto expand_row = [&](uint8_t* row, float scale) {     // this lane's row: codes -> bf16, front to back
#pragma unroll
    for (int c = 0; c < kByteChunks; ++c) {
      const uint4 codes = *reinterpret_cast<const uint4*>(row + D + c * 16);
      uint4 lo, hi;
      dequant16(codes, scale, lo, hi);
      *reinterpret_cast<uint4*>(row + c * 32) = lo;
      *reinterpret_cast<uint4*>(row + c * 32 + 16) = hi;
    }
  };
  int next_slots = -1;
  if (t0 + warp < t1) {
    next_slots = slot_of(t0 + warp);
    if (!KV8) {
      copy_rows(sk, p.k_cache, next_slots);
      copy_rows(sv, p.v_cache, next_slots);
    } else {
      copy_codes(sk, p.k_cache, next_slots);
      copy_codes(sv, p.v_cache, next_slots);
    }
  }

  for (int t = t0 + warp; t < t1; t += kDecWarps) {
    const int key0 = t * kDecTile;
    // int8 cache: this lane's row scales (0 for a key past the end: the codes are zeros there anyway)
    float ks = 0.f, vs = 0.f;
    if (KV8 && next_slots >= 0) {
      ks = p.k_scale[size_t(next_slots) * p.Hkv + kvh];
      vs = p.v_scale[size_t(next_slots) * p.Hkv + kvh];
    }
    cp_async_wait_but_one();                             // this tile's keys have landed; its values may still fly
    __syncwarp();
    if (KV8) {
      expand_row(sk + lane * kRow, ks);
      __syncwarp();
    }
    // ---- S[16 x 32] = Q · K^T: 4 n-tiles of 8 keys
    float s[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int ks = 0; ks < KS; ks += 2) {
        // matrices: (keys n*8.., d ks*16 + 0..7), (.., +8..15), (.., (ks+1)*16 + 0..7), (.., +8..15)
        uint32_t kb[4];
        ldmatrix_x4(kb, sk + (n * 8 + (lane & 7)) * kRow + ks * 32 + (lane >> 3) * 16);
        mma_bf16_16816(s[n], qa[ks], kb[0], kb[1]);
        mma_bf16_16816(s[n], qa[ks + 1], kb[2], kb[3]);
      }
    }
    __syncwarp();                                        // every lane has read this tile's keys
    next_slots = slot_of(t + kDecWarps);
    if (!KV8) copy_rows(sk, p.k_cache, next_slots);      // (an empty group when there is no next tile)
    else copy_codes(sk, p.k_cache, next_slots);
    // ---- mask, online softmax (log2 domain) for rows r0 = lane / 4 and r0 + 8
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int pos = key0 + n * 8 + 2 * (lane & 3) + j;
        const bool valid = pos < len && pos >= first_pos;
        s[n][j] = valid ? s[n][j] * p.scale_log2 : -INFINITY;
        s[n][2 + j] = valid ? s[n][2 + j] * p.scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, s[n][j]);
        mx1 = fmaxf(mx1, s[n][2 + j]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float a0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mn0);
    const float a1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mn1);
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pa[2][4];                                   // P as A fragments of the two 16-key k-steps
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const float p00 = (mn0 == -INFINITY) ? 0.f : exp2f(s[n][0] - mn0);
      const float p01 = (mn0 == -INFINITY) ? 0.f : exp2f(s[n][1] - mn0);
      const float p10 = (mn1 == -INFINITY) ? 0.f : exp2f(s[n][2] - mn1);
      const float p11 = (mn1 == -INFINITY) ? 0.f : exp2f(s[n][3] - mn1);
      sum0 += p00 + p01;
      sum1 += p10 + p11;
      pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16x2(p00, p01);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(p10, p11);
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * a0 + sum0;
    l1 = l1 * a1 + sum1;
    m0 = mn0;
    m1 = mn1;
#pragma unroll
    for (int n = 0; n < NT; ++n) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
    cp_async_wait_but_one();                             // this tile's values have landed; the next keys may still fly
    __syncwarp();
    if (KV8) {
      expand_row(sv + lane * kRow, vs);
      __syncwarp();
    }
    // ---- O[16 x D] += P[16 x 32] · V[32 x D]: V is [key][d], so its B fragments come through transposing loads
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        // matrices: (keys kk*16 + 0..7, d n*8..), (keys +8..15, d n*8..), (keys 0..7, d (n+1)*8..), (keys 8..15, ..)
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, sv + (kk * 16 + (lane & 15)) * kRow + (n + (lane >> 4)) * 16);
        mma_bf16_16816(o[n], pa[kk], vb[0], vb[1]);
        mma_bf16_16816(o[n + 1], pa[kk], vb[2], vb[3]);
      }
    }
    __syncwarp();
    if (!KV8) copy_rows(sv, p.v_cache, next_slots);      // every lane has read this tile's values
    else copy_codes(sv, p.v_cache, next_slots);
  }
  cp_async_wait_all();

  // ---- combine the 4 warps of the CTA (in warp order), then write the split's partial or the final output
  // smerge layout: [warp][16][D + 2], over the tiles: nobody may still be reading a tile
  __syncthreads();
  {
    const int r0 = lane >> 2, c0 = 2 * (lane & 3);
    float* d0 = smerge + (size_t(warp) * 16 + r0) * (D + 2);
    float* d1 = smerge + (size_t(warp) * 16 + r0 + 8) * (D + 2);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      d0[n * 8 + c0] = o[n][0]; d0[n * 8 + c0 + 1] = o[n][1];
      d1[n * 8 + c0] = o[n][2]; d1[n * 8 + c0 + 1] = o[n][3];
    }
    if ((lane & 3) == 0) { d0[D] = m0; d0[D + 1] = l0; d1[D] = m1; d1[D + 1] = l1; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, smerge[(size_t(w) * 16 + g) * (D + 2) + D]);
    float ll = 0.f, oo = 0.f;
    for (int w = 0; w < kDecWarps; ++w) {
      const float* src = smerge + (size_t(w) * 16 + g) * (D + 2);
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
  pdl_launch_dependents();     // a dependent launched programmatically may set itself up while this kernel runs
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
  const size_t tiles = size_t(kDecWarps) * 2 * kDecTile * (D * 2 + 16);
  const size_t merge = size_t(kDecWarps) * 16 * (D + 2) * 4;
  return size_t(16) * (D * 2 + 16) + (tiles > merge ? tiles : merge);
}

}  // namespace idrak

using namespace idrak;

IDRAK_API long long idrak_decode_partial_floats(int seqs, int H, int D, int splits) {
  return splits > 1 ? (long long)seqs * H * splits * (D + 2) : 0;
}

// The same over an int8 cache when k_scale / v_scale are given (one fp32 scale per (slot, kv head)).
IDRAK_API int idrak_paged_decode_kv(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                    const float* k_scale, const float* v_scale, const int* block_table,
                                    const int* seq_lens, void* out, float* partial, int seqs, int H, int Hkv, int D,
                                    int block_size, int max_blocks, int splits, float scale, int window, void* stream_) {
  if (D != 64 && D != 128) return -2;
  const bool kv8 = k_scale != nullptr;
  if (kv8 && !v_scale) return -6;
  if (H % Hkv || H / Hkv > kDecMaxGroup) return -3;
  if (splits > 1 && !partial) return -4;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride > 0 ? q_stride : (long long)H * D;
  if ((p.q_stride % 8) || (reinterpret_cast<uintptr_t>(q) & 15)) return -5;
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.partial = partial;
  p.H = H; p.Hkv = Hkv; p.D = D; p.block_size = block_size; p.max_blocks = max_blocks;
  p.splits = splits < 1 ? 1 : splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  dim3 grid(seqs, Hkv, p.splits);
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        cudaError_t e1 = cudaFuncSetAttribute(paged_decode_kernel<64, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              int(decode_smem<64>()));
        if (e1 == cudaSuccess)
          e1 = cudaFuncSetAttribute(paged_decode_kernel<64, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    int(decode_smem<64>()));
        if (e1 == cudaSuccess)
          e1 = cudaFuncSetAttribute(paged_decode_kernel<128, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    int(decode_smem<128>()));
        if (e1 == cudaSuccess)
          e1 = cudaFuncSetAttribute(paged_decode_kernel<128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    int(decode_smem<128>()));
        return int(e1);
      }))
    return e;
  if (D == 64) {
    if (kv8) paged_decode_kernel<64, 1><<<grid, kDecWarps * 32, decode_smem<64>(), s>>>(p);
    else paged_decode_kernel<64, 0><<<grid, kDecWarps * 32, decode_smem<64>(), s>>>(p);
  } else {
    if (kv8) paged_decode_kernel<128, 1><<<grid, kDecWarps * 32, decode_smem<128>(), s>>>(p);
    else paged_decode_kernel<128, 0><<<grid, kDecWarps * 32, decode_smem<128>(), s>>>(p);
  }
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

IDRAK_API int idrak_paged_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                                 const int* seq_lens, void* out, float* partial, int seqs, int H, int Hkv, int D,
                                 int block_size, int max_blocks, int splits, float scale, int window, void* stream_) {
  return idrak_paged_decode_kv(q, q_stride, k_cache, v_cache, nullptr, nullptr, block_table, seq_lens, out, partial, seqs,
                               H, Hkv, D, block_size, max_blocks, splits, scale, window, stream_);
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
