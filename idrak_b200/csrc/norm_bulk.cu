// LayerNorm / RMSNorm backward as a bulk-copy pipeline, for rows of 256 to 1024 elements.
//
// The plain kernel (rowops.cu: one warp per row, operands loaded into registers) keeps too few bytes in flight per
// SM to reach HBM speed and spends most of its registers on per-column accumulators. Here one CTA per SM runs a
// producer thread that streams chunks of consecutive rows of dy, x and the residual gradient into a ring of
// shared-memory stages with cp.async.bulk (rows are contiguous, so a chunk of one operand is one copy), completing
// on an mbarrier per stage, while twelve consumer warps work on the landed stage.
//
// The consumer warps form G groups of W = ceil(C / 256) warps; a lane owns eight consecutive columns (one 128-bit
// shared-memory load per operand and row) and a group takes two rows of every stage:
//   phase A  the lane's share of s1 = sum(dy w) and s2 = sum(dy w n) of its two rows, a six-shuffle reduction over
//            the warp, the warps of the group combined through shared memory behind a group-wide named barrier;
//   phase B  dx = (dy w - s1 - n s2) rstd (+ residual gradient) stored with one 128-bit store, and the lane's
//            eight columns of d(weight), d(bias) and - new - of the column sums of dx accumulated in registers.
// At the end the groups' accumulators are folded in group order through shared memory, so every sum has a fixed
// order (rows ascending inside a group, groups ascending, then colsum_final_kernel over the CTAs in CTA order).
// dx of a pre-norm block is the gradient of the preceding linear layer's output, so its column sums are that
// layer's bias gradient and the separate column-sum pass over dx disappears. Every wait is bounded and reports
// through the status word.
//
// Reference counterparts: layernorm_bwd_f32 / layernorm_bwd_params_f32 (src/Idrak.Gpu/Cuda/PtxKernels.Decoding.cs:12),
// rms_norm_backward_f32 (PtxKernels.Decoder.cs:14).
#include "norm_bulk.h"

namespace idrak {

constexpr int kNbWarps = 12;               // consumer warps
constexpr int kNbThreads = 32 * (kNbWarps + 1);

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void unpack8(const uint4& a, float (&v)[8]) {
  float2 f;
  f = unpack_bf16x2(a.x); v[0] = f.x; v[1] = f.y;
  f = unpack_bf16x2(a.y); v[2] = f.x; v[3] = f.y;
  f = unpack_bf16x2(a.z); v[4] = f.x; v[5] = f.y;
  f = unpack_bf16x2(a.w); v[6] = f.x; v[7] = f.y;
}

// Four per-lane values -> the warp's four totals: lane L ends up with the total of value 2 * bit4(L) + bit3(L).
__device__ __forceinline__ float warp_reduce4(float v0, float v1, float v2, float v3, int lane) {
  const bool hi16 = (lane & 16) != 0;
  float a = hi16 ? v2 : v0, b = hi16 ? v3 : v1;               // what this lane keeps
  const float sa = hi16 ? v0 : v2, sb = hi16 ? v1 : v3;       // what its partner keeps
  a += __shfl_xor_sync(0xffffffffu, sa, 16);
  b += __shfl_xor_sync(0xffffffffu, sb, 16);
  const bool hi8 = (lane & 8) != 0;
  float c = hi8 ? b : a;
  const float sc = hi8 ? a : b;
  c += __shfl_xor_sync(0xffffffffu, sc, 8);
  c += __shfl_xor_sync(0xffffffffu, c, 4);
  c += __shfl_xor_sync(0xffffffffu, c, 2);
  c += __shfl_xor_sync(0xffffffffu, c, 1);
  return c;
}

__global__ void __launch_bounds__(kNbThreads, 1) norm_bwd_bulk_kernel(const NormBulkParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int C = p.C;
  const int nvec = C >> 3;
  const int narr = p.dres ? 3 : 2;
  const int wpr = (nvec + 31) >> 5;                       // warps per row group: 1..4
  const int groups = kNbWarps / wpr;                      // 12, 6, 4 or 3
  const int srows = 2 * groups;                           // rows per stage
  const uint32_t arr_bytes = uint32_t(srows) * C * 2;
  const uint32_t stage_bytes = arr_bytes * narr;
  float4* red = reinterpret_cast<float4*>(smem + size_t(p.stages) * stage_bytes);   // [2][kNbWarps]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + 2 * kNbWarps);
  uint64_t* empty = full + p.stages;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(empty + p.stages);

  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * p.rows_per_block;
  const int row1 = min(p.rows, row0 + p.rows_per_block);
  const int chunks = row1 > row0 ? (row1 - row0 + srows - 1) / srows : 0;
  const int used_warps = groups * wpr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], used_warps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();

  if (wid == kNbWarps) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, issued_phase = 0;
      bool ok = true;
      for (int c = 0; c < chunks && ok; ++c) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (9u << 16) | stage)) {
          ok = false;
          break;
        }
        const int r = row0 + c * srows;
        const uint32_t bytes = uint32_t(min(srows, row1 - r)) * C * 2;
        uint8_t* s = smem + size_t(stage) * stage_bytes;
        mbar_expect_tx(&full[stage], bytes * narr);
        bulk_load(s, p.dy + size_t(r) * C, bytes, &full[stage]);
        bulk_load(s + arr_bytes, p.x + size_t(r) * C, bytes, &full[stage]);
        if (p.dres) bulk_load(s + 2 * arr_bytes, p.dres + size_t(r) * C, bytes, &full[stage]);
        issued_mask |= 1u << stage;
        issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (!ok || *abort_flag) {
        // give up: let the copies already issued land before the CTA's shared memory goes away
        for (int s = 0; s < p.stages; ++s) {
          if (issued_mask & (1u << s)) {
            const uint32_t par = (issued_phase >> s) & 1u;
            for (int i = 0; i < (1 << 20); ++i)
              if (mbar_try_wait(&full[s], par)) break;
          }
        }
      }
    }
  }

  // -------------------------------------------------------------------- consumers
  const bool consumer = wid < used_warps;
  const int grp = wid / wpr, sub = wid - grp * wpr;
  const int vi = sub * 32 + lane;                         // this lane's vector (8 columns) of the row
  const bool live = consumer && vi < nvec;
  float dw[8], db[8], ds[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { dw[j] = 0.f; db[j] = 0.f; ds[j] = 0.f; }
  if (consumer) {
    float w8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w8[j] = 0.f;
    if (live) unpack8(*reinterpret_cast<const uint4*>(p.w + vi * 8), w8);
    const float inv_c = 1.f / float(C);
    const int gthreads = wpr * 32;
    int stage = 0;
    uint32_t phase = 0;
    for (int c = 0; c < chunks; ++c) {
      const int ra = row0 + c * srows + 2 * grp;          // this group's two rows of the chunk
      const bool va = ra < row1, vb = ra + 1 < row1;
      // per-row scalars (one address for the whole warp) while the stage is still landing
      const float rstd_a = va ? p.rstd[ra] : 0.f, rstd_b = vb ? p.rstd[ra + 1] : 0.f;
      const float shift_a = (va && !p.rms) ? -p.mean[ra] * rstd_a : 0.f;
      const float shift_b = (vb && !p.rms) ? -p.mean[ra + 1] * rstd_b : 0.f;
      if (!mbar_wait(&full[stage], phase, abort_flag, p.st, kTimeoutSmemFull, (9u << 16) | stage)) break;
      const uint8_t* s = smem + size_t(stage) * stage_bytes + size_t(2 * grp) * C * 2;
      const uint4* sdy = reinterpret_cast<const uint4*>(s) + vi;
      const uint4* sx = reinterpret_cast<const uint4*>(s + arr_bytes) + vi;
      const uint4* sdr = reinterpret_cast<const uint4*>(s + 2 * arr_bytes) + vi;
      // ---- phase A
      float dy[2][8], g[2][8], n[2][8];
      float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const bool valid = live && (r == 0 ? va : vb);
        const float rstd = r == 0 ? rstd_a : rstd_b, shift = r == 0 ? shift_a : shift_b;
        if (valid) {
          float xv[8];
          unpack8(sdy[r * nvec], dy[r]);
          unpack8(sx[r * nvec], xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            n[r][j] = fmaf(xv[j], rstd, shift);
            g[r][j] = dy[r][j] * w8[j];
            part[2 * r] += g[r][j];
            part[2 * r + 1] = fmaf(g[r][j], n[r][j], part[2 * r + 1]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) { dy[r][j] = 0.f; g[r][j] = 0.f; n[r][j] = 0.f; }
        }
      }
      const float mine = warp_reduce4(part[0], part[1], part[2], part[3], lane);
      // lanes 0, 8, 16, 24 hold totals 0..3 of this warp
      float* slot = reinterpret_cast<float*>(red + (c & 1) * kNbWarps + wid);
      if ((lane & 7) == 0) slot[lane >> 3] = mine;
      named_sync(1 + grp, gthreads);
      float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int w = 0; w < wpr; ++w) {                     // warp order: the same sum in every lane of the group
        const float4 t = red[(c & 1) * kNbWarps + grp * wpr + w];
        tot.x += t.x; tot.y += t.y; tot.z += t.z; tot.w += t.w;
      }
      // ---- phase B
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const bool valid = live && (r == 0 ? va : vb);
        if (valid) {
          const float rstd = r == 0 ? rstd_a : rstd_b;
          const float s1 = p.rms ? 0.f : (r == 0 ? tot.x : tot.z) * inv_c;
          const float s2 = (r == 0 ? tot.y : tot.w) * inv_c;
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (g[r][j] - s1 - n[r][j] * s2) * rstd;
          if (p.dres) {
            float r8[8];
            unpack8(sdr[r * nvec], r8);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += r8[j];
          }
          uint4 pk;
          pk.x = pack_bf16x2(o[0], o[1]); pk.y = pack_bf16x2(o[2], o[3]);
          pk.z = pack_bf16x2(o[4], o[5]); pk.w = pack_bf16x2(o[6], o[7]);
          *reinterpret_cast<uint4*>(p.dx + size_t(ra + r) * C + vi * 8) = pk;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            dw[j] = fmaf(dy[r][j], n[r][j], dw[j]);
            db[j] += dy[r][j];
          }
          if (p.dxs_part) {
            // the sum of what was stored (bf16), as a separate column-sum pass over dx would see it
            float q[8];
            unpack8(pk, q);
#pragma unroll
            for (int j = 0; j < 8; ++j) ds[j] += q[j];
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
      if (++stage == p.stages) { stage = 0; phase ^= 1; }
    }
  }

  // ---- fold the groups' column sums in group order (the stages are free now: every copy was consumed or waited for)
  __syncthreads();
  float* acc = reinterpret_cast<float*>(smem);            // [3][C]
  for (int i = threadIdx.x; i < 3 * C; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  for (int gsel = 0; gsel < groups; ++gsel) {
    if (live && grp == gsel) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[vi * 8 + j] += dw[j];
        acc[C + vi * 8 + j] += db[j];
        acc[2 * C + vi * 8 + j] += ds[j];
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    p.dw_part[size_t(blockIdx.x) * C + i] = acc[i];
    if (p.db_part) p.db_part[size_t(blockIdx.x) * C + i] = acc[C + i];
    if (p.dxs_part) p.dxs_part[size_t(blockIdx.x) * C + i] = acc[2 * C + i];
  }
}

static inline int stage_rows(int C) {
  const int wpr = (C / 8 + 31) / 32;
  return 2 * (kNbWarps / wpr);
}

// How many CTAs / partial rows a call of these sizes uses (0: the sizes do not fit this kernel).
int norm_bwd_bulk_blocks(int rows, int C) {
  if (C % 8 || C < 256 || C > 1024 || rows < 64) return 0;
  const int sms = sm_count();
  const int sr = stage_rows(C);
  const int by_rows = (rows + sr - 1) / sr;
  return by_rows < sms ? by_rows : sms;
}

int norm_bwd_bulk_launch(const NormBulkParams& base, int blocks, cudaStream_t stream) {
  NormBulkParams p = base;
  const int narr = p.dres ? 3 : 2;
  const int sr = stage_rows(p.C);
  const size_t stage_bytes = size_t(sr) * p.C * 2 * narr;
  const size_t budget = 216 * 1024;
  int stages = int(budget / stage_bytes);
  if (stages > 8) stages = 8;
  if (stages < 2) return -2;
  // rows per CTA: a multiple of the chunk so only the last CTA sees a ragged chunk
  int rpb = (p.rows + blocks - 1) / blocks;
  rpb = (rpb + sr - 1) / sr * sr;
  p.rows_per_block = rpb;
  p.stages = stages;
  p.st = status_device_ptr();
  size_t smem = stages * stage_bytes + size_t(2) * kNbWarps * sizeof(float4) + 2 * stages * sizeof(uint64_t) + 16 + 128;
  const size_t fold = size_t(3) * p.C * sizeof(float) + 128;
  if (smem < fold) smem = fold;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(norm_bwd_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
      }))
    return e;
  norm_bwd_bulk_kernel<<<blocks, kNbThreads, smem, stream>>>(p);
  note_launches(1);
  return int(cudaGetLastError());
}

}  // namespace idrak
