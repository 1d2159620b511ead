// Flash attention backward for sm_100a, as two deterministic kernels (no float atomics):
//
//   flash_bwd_q   one CTA per 128 query rows of a (batch, head): for each key block recompute
//                 S = Q K^T and dP = dO V^T into TMEM, form dS = P * (dP - delta) * scale in registers,
//                 stage it as a bf16 operand and accumulate dQ += dS K in TMEM.
//   flash_bwd_kv  one CTA per 128 keys of a (batch, kv head): for every query head of the group and every
//                 query block that can see these keys recompute S^T = K Q^T and dP^T = V dO^T (so a
//                 thread owns a key row), form P^T and dS^T, and accumulate dV += P^T dO and
//                 dK += dS^T Q in TMEM. Grouped-query heads are summed inside the CTA.
//   flash_delta   delta[b,h,s] = sum_d dO * O.
//
// Warp roles match the forward kernel: warp 0 feeds shared memory with TMA, warp 1 issues tcgen05.mma,
// warps 2..9 do the element-wise work, two threads per tile row with 64 of the block's 128 columns each (the row
// statistics come from the forward pass, so the halves are independent). The operand tiles the element-wise warps
// produce (dS; P^T and dS^T) are double-buffered, each buffer with its own "product done" barrier, so the next block is
// filled while the tensor cores still accumulate from the previous one. The same 128B-swizzled tile serves as a
// K-major operand for one product and as an MN-major operand for the other, so nothing is transposed.
//
// Reference counterparts: flash_tc_bwd_q_d{64,128}, flash_tc_bwd_kv_d{64,128}, flash_tc_delta
// (src/Idrak.Gpu/Cuda/PtxKernels.FlashTensorCore.cs) and attn_bwd_{d,kv,q}_f32 (PtxKernels.Rows.cs:1222-1750).
#include "flash_common.cuh"

namespace idrak {

constexpr float kLog2e = 1.4426950408889634f;

constexpr int kBwdThreads = 320;      // TMA warp, MMA warp, eight element-wise warps (two threads per tile row)
__device__ __forceinline__ void softmax_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Write 32 consecutive columns [c*32, c*32+32) of row r of a 128x128 bf16 K-major operand tile.
__device__ __forceinline__ void store_operand_chunk(uint8_t* tile, int r, int c, const float (&v)[32]) {
  uint8_t* atom = tile + (c >> 1) * 16384 + r * 128;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int chunk = ((c & 1) * 4 + g) ^ (r & 7);
    uint4 o;
    o.x = pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]);
    o.y = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
    o.z = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]);
    o.w = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
    *reinterpret_cast<uint4*>(atom + chunk * 16) = o;
  }
}

// K-major operand tile [128 rows][D]: descriptor for k-step kk (16 columns)
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, int kk) {
  return make_smem_desc_sw128(base + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
}
// The same tile read as an MN-major operand (N = D, contraction over its 128 rows): k-step kk = 16 rows
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t base, int kk) {
  return make_smem_desc_sw128(base + kk * 2048, 16384, 1024);
}

// ---------------------------------------------------------------------------
// delta
// ---------------------------------------------------------------------------
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dO,
                                   float* __restrict__ delta, int B, int S, int H, int D) {
  // D/8 lanes share one (b, s, h) row, each with one 128-bit load of O and of dO; a warp covers 256/D rows
  const int lanes_per_row = D >> 3;
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long w = t / lanes_per_row;
  const int sub = int(t - w * lanes_per_row);
  const long long total = (long long)B * S * H;
  float acc = 0.f;
  if (w < total) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + w * D + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(dO + w * D + sub * 8);
    float2 x, y;
    x = unpack_bf16x2(a.x); y = unpack_bf16x2(g.x); acc += x.x * y.x + x.y * y.y;
    x = unpack_bf16x2(a.y); y = unpack_bf16x2(g.y); acc += x.x * y.x + x.y * y.y;
    x = unpack_bf16x2(a.z); y = unpack_bf16x2(g.z); acc += x.x * y.x + x.y * y.y;
    x = unpack_bf16x2(a.w); y = unpack_bf16x2(g.w); acc += x.x * y.x + x.y * y.y;
  }
  for (int o2 = lanes_per_row >> 1; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
  if (w < total && sub == 0) {
    const int h = int(w % H);
    const long long bs = w / H;
    const int s = int(bs % S);
    const int b = int(bs / S);
    delta[((long long)b * H + h) * S + s] = acc;
  }
}

// ---------------------------------------------------------------------------
// dQ
// ---------------------------------------------------------------------------
template <int D>
struct BwdQSmem {
  static constexpr int kTile = 128 * D * 2;
  // three K / V stages at head size 64: a stage is freed only by the dQ product of its block, and with two the load of
  // block j + 2 (about 1500 cycles from L2) sat on the critical path of every block
  static constexpr int kStages = (D == 64) ? 3 : 1;
  static constexpr int kQ = 0;
  static constexpr int kDO = kQ + kTile;
  static constexpr int kK = kDO + kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kDS = kV + kStages * kTile;          // two dS tiles: the next one is filled while the tensor
  static constexpr int kBar = kDS + 2 * 32768;              // cores still read the previous one for dQ
  static constexpr int kTotal = kBar + 256 + 1024;
};

// Persistent, like the dK / dV kernel below: one CTA per SM walks (query block, head, batch) units, heaviest first; the
// next unit's Q and dO load while the current unit's last block is in its element-wise and dQ steps, and the write-out of
// dQ overlaps the next unit's first score products.
// Unit `round` of this CTA. The units are sorted heaviest first; the CTAs take them in rounds, forwards in even rounds and
// backwards in odd ones, so a CTA that drew a heavier unit than its neighbours in one round draws a lighter one in the
// next (the static counterpart of handing units out one by one).
__device__ __forceinline__ int snake_unit(int round, int units) {
  const int g = int(gridDim.x), c = int(blockIdx.x);
  const int u = round * g + ((round & 1) ? (g - 1 - c) : c);
  return u < units ? u : -1;
}
__device__ __forceinline__ int snake_rounds(int units) { return (units + int(gridDim.x) - 1) / int(gridDim.x); }

struct QUnit {
  int qb, head, batch, kv_head, q0, jlo, nkv;
};

template <bool MODES>
__device__ __forceinline__ QUnit q_unit(const FlashParams& p, int u, int off, int nqt) {
  QUnit t;
  const int per_qb = p.H * p.B;
  const int slot = u / per_qb;
  t.qb = p.causal ? (nqt - 1 - slot) : slot;      // later query blocks see more keys: they go first
  const int rem = u - slot * per_qb;
  t.head = rem % p.H;
  t.batch = rem / p.H;
  t.kv_head = t.head / (p.H / p.Hkv);
  t.q0 = t.qb * 128;
  int nkv_end = (p.Skv + 127) / 128;
  if (p.causal) nkv_end = min(nkv_end, (t.q0 + 127 + off) / 128 + 1);
  if (nkv_end < 0) nkv_end = 0;
  // key blocks wholly below what the tile's first row may see are skipped (window / packed-sequence bounds)
  const bool bounded = MODES && p.causal && (p.window > 0 || p.row_start != nullptr);
  t.jlo = bounded ? min(nkv_end, max(0, flash_row_lo(p, t.batch, min(t.q0, p.Sq - 1), off)) / 128) : 0;
  t.nkv = nkv_end - t.jlo;      // key block of iteration j is jlo + j
  return t;
}

template <int D, bool MODES>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_q_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const FlashParams p) {
  using L = BwdQSmem<D>;
  constexpr int NS = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* qdo_full = bars + 0;
  uint64_t* kv_full = bars + 1;     // [3]
  uint64_t* kv_empty = bars + 4;    // [3]
  uint64_t* sdp_full = bars + 7;
  uint64_t* ds_ready = bars + 8;
  uint64_t* dq_done = bars + 9;     // [2]: one per dS tile
  uint64_t* sdp_taken = bars + 11;  // the element-wise warps hold S and dP of the block in registers: TMEM may be rewritten
  uint64_t* qdo_free = bars + 12;   // the unit's last score products have read Q and dO: the next unit's may land
  uint64_t* dq_free = bars + 13;    // dQ of the unit sits in registers: the next unit may accumulate
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int off = p.Skv - p.Sq;
  const int nqt = (p.Sq + 127) / 128;
  const int units = nqt * p.H * p.B;
  const bool bounded = MODES && p.causal && (p.window > 0 || p.row_start != nullptr);

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(ds_ready, 256);
    mbar_init(&dq_done[0], 1);
    mbar_init(&dq_done[1], 1);
    mbar_init(sdp_taken, 256);
    mbar_init(qdo_free, 1);
    mbar_init(dq_free, 256);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
  }
  constexpr uint32_t kTmemCols = 512;   // S [0,128) | dP [128,256) | dQ [256, 256+D)
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dQ = tmem_base + 256;

  // Every role walks the same units and counts alike: n = units with work so far, g = key blocks so far over all units.
  if (warp == 0) {
    if (lane == 0) {
      int n = 0, g = 0;
      bool ok = true;
      for (int round = 0; round < snake_rounds(units) && ok; ++round) {
        const int u = snake_unit(round, units);
        if (u < 0) continue;
        const QUnit t = q_unit<MODES>(p, u, off, nqt);
        if (t.nkv <= 0) continue;
        if (n > 0 && !mbar_wait(qdo_free, (n - 1) & 1, abort_flag, p.st, kTimeoutSmemEmpty, (3u << 16) | 14)) break;
        mbar_expect_tx(qdo_full, 2 * L::kTile);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_4d(smem + L::kQ + c * 16384, &tmQ, qdo_full, c * 64, t.q0, t.head, t.batch);
          tma_load_4d(smem + L::kDO + c * 16384, &tmDO, qdo_full, c * 64, t.q0, t.head, t.batch);
        }
        for (int j = 0; j < t.nkv; ++j, ++g) {
          const int st = g % NS;
          const uint32_t ph = (g / NS) & 1;
          if (!mbar_wait(&kv_empty[st], ph ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (3u << 16) | st)) { ok = false; break; }
          mbar_expect_tx(&kv_full[st], 2 * L::kTile);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            tma_load_4d(smem + L::kK + st * L::kTile + c * 16384, &tmK, &kv_full[st], c * 64, (t.jlo + j) * 128, t.kv_head, t.batch);
            tma_load_4d(smem + L::kV + st * L::kTile + c * 16384, &tmV, &kv_full[st], c * 64, (t.jlo + j) * 128, t.kv_head, t.batch);
          }
        }
        ++n;
      }
      if (*abort_flag) __nanosleep(50000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(128, 128, 0, 0, 1);
      constexpr uint32_t idesc_dq = make_idesc_f16(128, D, 0, 1, 1);
      const uint32_t sq = smem_u32(smem + L::kQ), sdo = smem_u32(smem + L::kDO), sds = smem_u32(smem + L::kDS);
      int n = 0, g0 = 0;
      bool ok = true;
      // S and dP of global block g; within a unit they are issued one block ahead, as soon as the element-wise warps
      // have taken the previous block's S and dP into registers
      auto issue_scores = [&](int g) -> bool {
        const int st = g % NS;
        const uint32_t ph = (g / NS) & 1;
        if (!mbar_wait(&kv_full[st], ph, abort_flag, p.st, kTimeoutSmemFull, (3u << 16) | st)) return false;
        if (g > 0 && !mbar_wait(sdp_taken, (g - 1) & 1, abort_flag, p.st, kTimeoutTmemEmpty, (3u << 16) | 13)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + L::kK + st * L::kTile), sv = smem_u32(smem + L::kV + st * L::kTile);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc_mma_f16_ss(tmem_S, kmajor_desc(sq, kk), kmajor_desc(sk, kk), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc_mma_f16_ss(tmem_dP, kmajor_desc(sdo, kk), kmajor_desc(sv, kk), idesc_s, kk > 0 ? 1u : 0u);
        tc_commit(sdp_full);
        return true;
      };
      constexpr bool kAhead = NS >= 2;      // one stage: the next K / V cannot land before this block's dQ product is done
      for (int round = 0; round < snake_rounds(units) && ok; ++round) {
        const int u = snake_unit(round, units);
        if (u < 0) continue;
        const QUnit t = q_unit<MODES>(p, u, off, nqt);
        if (t.nkv <= 0) continue;
        if (!mbar_wait(qdo_full, n & 1, abort_flag, p.st, kTimeoutSmemFull, (3u << 16) | 8)) break;
        if (kAhead) {
          ok = issue_scores(g0);
          if (ok && t.nkv == 1) tc_commit(qdo_free);
        }
        for (int j = 0; j < t.nkv && ok; ++j) {
          const int g = g0 + j;
          const int st = g % NS;
          if (kAhead) {
            if (j + 1 < t.nkv) {
              if (!issue_scores(g + 1)) { ok = false; break; }
              if (j + 2 == t.nkv) tc_commit(qdo_free);        // the unit's last score products are on their way
            }
          } else {
            if (!issue_scores(g)) { ok = false; break; }
            if (j + 1 == t.nkv) tc_commit(qdo_free);
          }
          if (!mbar_wait(ds_ready, g & 1, abort_flag, p.st, kTimeoutGeneric, (3u << 16) | 9)) { ok = false; break; }
          if (j == 0 && n > 0) {
            // dQ of the previous unit must have been read out before this unit starts its own sum
            if (!mbar_wait(dq_free, (n - 1) & 1, abort_flag, p.st, kTimeoutTmemEmpty, (3u << 16) | 15)) { ok = false; break; }
          }
          tc_fence_after();
          const uint32_t sk = smem_u32(smem + L::kK + st * L::kTile);
          const uint32_t sds_b = sds + (g & 1) * 32768;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            tc_mma_f16_ss(tmem_dQ, kmajor_desc(sds_b, kk), mnmajor_desc(sk, kk), idesc_dq, (j > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&kv_empty[st]);
          tc_commit(&dq_done[g & 1]);
        }
        g0 += t.nkv;
        ++n;
      }
    }
  } else {
    // Two threads per query row: warps 2..5 take key columns [0, 64) of a block, warps 6..9 columns [64, 128); the
    // row's statistics come from the forward pass, so the halves are independent.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const bool capped = MODES && p.softcap > 0.f;
    const bool special = bounded || capped;
    const float cap_in = capped ? p.scale / p.softcap : 0.f;
    const float cap_l2 = p.softcap * kLog2e;
    constexpr int kOC = D / 2;               // each half writes D / 2 columns of the row
    int g0 = 0;
    bool ok = true;
    for (int round = 0; round < snake_rounds(units) && ok; ++round) {
      const int u = snake_unit(round, units);
      if (u < 0) continue;
      const QUnit t = q_unit<MODES>(p, u, off, nqt);
      const int row = t.q0 + r;
      __nv_bfloat16* drow = p.dQ + (size_t(t.batch) * p.Sq + row) * p.dq_row_stride + size_t(t.head) * D + half * kOC;
      if (t.nkv <= 0) {
        if (row < p.Sq)
          for (int i = 0; i < kOC; i += 8) *reinterpret_cast<uint4*>(drow + i) = make_uint4(0, 0, 0, 0);
        continue;
      }
      float lse2 = INFINITY, dlt = 0.f;
      if (row < p.Sq) {
        const size_t idx = (size_t(t.batch) * p.H + t.head) * p.Sq + row;
        const float l = p.lse[idx];
        lse2 = (l == -INFINITY) ? INFINITY : l * kLog2e;
        dlt = p.delta[idx];
      }
      const int row_lo = bounded ? flash_row_lo(p, t.batch, row, off) : 0;
      for (int j = 0; j < t.nkv && ok; ++j) {
        const int g = g0 + j;
        if (!mbar_wait(sdp_full, g & 1, abort_flag, p.st, kTimeoutTmemFull, (3u << 16) | 10)) { ok = false; break; }
        tc_fence_after();
        uint8_t* sDS = smem + L::kDS + (g & 1) * 32768;
        const int k0 = (t.jlo + j) * 128 + half * 64;          // first key of this thread's 64 columns
        int lim = p.Skv - k0;
        if (p.causal) lim = min(lim, row + off - k0 + 1);
        lim = max(0, min(64, lim));
        const int lo = max(0, min(64, row_lo - k0));           // keys below the row's window / sequence start
        // four loads in flight and one wait; once every thread holds its part the MMA warp may overwrite S and dP with
        // the next block's
        uint32_t s[2][32], dp[2][32];
        tmem_ld_32x32b_x32(tmem_S + lane_addr + half * 64, s[0]);
        tmem_ld_32x32b_x32(tmem_S + lane_addr + half * 64 + 32, s[1]);
        tmem_ld_32x32b_x32(tmem_dP + lane_addr + half * 64, dp[0]);
        tmem_ld_32x32b_x32(tmem_dP + lane_addr + half * 64 + 32, dp[1]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(sdp_taken);
        if (g >= 2) {
          // the dQ product that last read this dS tile (block g - 2) must be complete
          if (!mbar_wait(&dq_done[g & 1], uint32_t((g >> 1) - 1) & 1u, abort_flag, p.st, kTimeoutTmemFull, (3u << 16) | 11)) {
            ok = false;
            break;
          }
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          float ds[32];
          if (!special) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float pr = fast_exp2(__uint_as_float(s[cc][i]) * p.scale_log2 - lse2);
              float v = pr * (__uint_as_float(dp[cc][i]) - dlt) * p.scale;
              ds[i] = (cc * 32 + i < lim) ? v : 0.f;
            }
          } else {
            // lower key bound and / or soft-capped scores: u = cap * tanh(s * scale / cap), du/ds = scale * (1 - tanh^2)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float sc = __uint_as_float(s[cc][i]), gr = p.scale;
              if (capped) {
                const float th = tanh_fast(sc * cap_in);
                sc = th * cap_l2;
                gr *= 1.f - th * th;
              } else {
                sc *= p.scale_log2;
              }
              float pr = fast_exp2(sc - lse2);
              float v = pr * (__uint_as_float(dp[cc][i]) - dlt) * gr;
              ds[i] = (cc * 32 + i < lim && cc * 32 + i >= lo) ? v : 0.f;
            }
          }
          store_operand_chunk(sDS, r, half * 2 + cc, ds);
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(ds_ready);
      }
      if (!ok) break;
      const int last = g0 + t.nkv - 1;
      if (!mbar_wait(&dq_done[last & 1], uint32_t(last >> 1) & 1u, abort_flag, p.st, kTimeoutTmemFull, (3u << 16) | 12)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // dQ leaves tensor memory first, so the next unit may start accumulating while the row is packed and stored
      uint32_t o[kOC];
#pragma unroll
      for (int c = 0; c < kOC / 32; ++c)
        tmem_ld_32x32b_x32(tmem_dQ + lane_addr + half * kOC + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&o[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_free);
      if (row < p.Sq) {
#pragma unroll
        for (int gq = 0; gq < kOC / 8; ++gq) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[gq * 8 + 0]), __uint_as_float(o[gq * 8 + 1]));
          w.y = pack_bf16x2(__uint_as_float(o[gq * 8 + 2]), __uint_as_float(o[gq * 8 + 3]));
          w.z = pack_bf16x2(__uint_as_float(o[gq * 8 + 4]), __uint_as_float(o[gq * 8 + 5]));
          w.w = pack_bf16x2(__uint_as_float(o[gq * 8 + 6]), __uint_as_float(o[gq * 8 + 7]));
          *reinterpret_cast<uint4*>(drow + gq * 8) = w;
        }
      }
      g0 += t.nkv;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// dK, dV
// ---------------------------------------------------------------------------
template <int D>
struct BwdKVSmem {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kStages = (D == 64) ? 2 : 1;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile;
  static constexpr int kQ = kV + kTile;
  static constexpr int kDO = kQ + kStages * kTile;
  // head size 64: two P^T / dS^T buffers, so the element-wise warps fill the next pair while the tensor cores still
  // accumulate dV / dK from the previous one (224 KB in all; at head size 128 there is room for one pair only)
  static constexpr int kPBufs = (D == 64) ? 2 : 1;
  static constexpr int kPT = kDO + kStages * kTile;
  static constexpr int kDST = kPT + kPBufs * 32768;
  static constexpr int kStat = kDST + kPBufs * 32768;       // lse2[128], delta[128], lo[128]
  static constexpr int kBar = kStat + 1536;
  static constexpr int kTotal = kBar + 256 + 1024;
};

// Persistent: the grid is one CTA per SM and every CTA walks a list of (key block, kv head, batch) units, heaviest
// first. Barriers, tensor memory and the Q / dO ring are set up once; the next unit's K and V load while the last block of
// the current unit is still in its element-wise and accumulation steps, and the write-out of dK / dV overlaps the first
// score products of the next unit. With one launch of 1536 short CTAs the set-up, first-load and write-out latencies
// (about 12 k cycles per CTA) ran unhidden, a third of the time at 1024 tokens.
struct KvUnit {
  int kb, kv_head, batch, k0, i_min, per_head, iters;
};

template <bool MODES>
__device__ __forceinline__ KvUnit kv_unit(const FlashParams& p, int u, int off, int nq) {
  KvUnit t;
  const int per_kb = p.Hkv * p.B;
  t.kb = u / per_kb;                         // ascending key block = most query blocks first under a causal mask
  const int rem = u - t.kb * per_kb;
  t.kv_head = rem % p.Hkv;
  t.batch = rem / p.Hkv;
  t.k0 = t.kb * 128;
  t.i_min = p.causal ? max(0, (t.k0 - off) / 128) : 0;
  // query blocks past the last one that can see these keys are skipped too: a sliding window bounds them directly,
  // packed sequences by the first block whose first row already starts beyond this key block
  int i_end = nq;
  if (MODES && p.causal && (p.window > 0 || p.row_start != nullptr)) {
    if (p.window > 0) i_end = min(i_end, (t.k0 + 127 + p.window - 1 - off) / 128 + 1);
    if (p.row_start) {
      int i = t.i_min;
      while (i < i_end && p.row_start[size_t(t.batch) * p.Sq + min(i * 128, p.Sq - 1)] <= t.k0 + 127) ++i;
      i_end = i;
    }
    i_end = max(i_end, t.i_min);
  }
  t.per_head = max(0, i_end - t.i_min);
  t.iters = t.per_head * (p.H / p.Hkv);
  return t;
}

template <int D, bool MODES>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_kv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const FlashParams p) {
  using L = BwdKVSmem<D>;
  constexpr int NS = L::kStages;
  constexpr int PB = L::kPBufs;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;    // [2]
  uint64_t* qdo_empty = bars + 3;   // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* pds_ready = bars + 6;
  uint64_t* acc_done = bars + 7;    // [2]: one per P^T / dS^T buffer
  uint64_t* sdp_taken = bars + 9;   // S^T and dP^T of the block are in registers: TMEM may be rewritten
  uint64_t* kv_free = bars + 10;    // the unit's last score products have read K and V: the next unit's may land
  uint64_t* acc_free = bars + 11;   // dV and dK of the unit sit in registers: the next unit may accumulate
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* s_lse2 = reinterpret_cast<float*>(smem + L::kStat);
  float* s_delta = s_lse2 + 128;
  int* s_lo = reinterpret_cast<int*>(s_delta + 128);      // first key each query of the block may see

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.H / p.Hkv;
  const int off = p.Skv - p.Sq;
  const int nq = (p.Sq + 127) / 128;
  const int units = ((p.Skv + 127) / 128) * p.Hkv * p.B;
  const bool bounded = MODES && p.causal && (p.window > 0 || p.row_start != nullptr);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 256);
    mbar_init(&acc_done[0], 1);
    mbar_init(&acc_done[1], 1);
    mbar_init(sdp_taken, 256);
    mbar_init(kv_free, 1);
    mbar_init(acc_free, 256);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
  }
  constexpr uint32_t kTmemCols = 512;   // S^T [0,128) | dP^T [128,256) | dV [256,256+D) | dK [256+D, 256+2D)
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_ST = tmem_base, tmem_dPT = tmem_base + 128, tmem_dV = tmem_base + 256,
                 tmem_dK = tmem_base + 256 + D;

  // Every role walks the same units and counts the same things: n = units with work so far (parity of the per-unit
  // barriers), g = query blocks so far over all units (stage and parity of the per-block barriers).
  if (warp == 0) {
    if (lane == 0) {
      int n = 0, g = 0;
      bool ok = true;
      for (int round = 0; round < snake_rounds(units) && ok; ++round) {
        const int u = snake_unit(round, units);
        if (u < 0) continue;
        const KvUnit t = kv_unit<MODES>(p, u, off, nq);
        if (t.iters == 0) continue;
        // K and V of this unit: once the previous unit's last score products have read theirs
        if (n > 0 && !mbar_wait(kv_free, (n - 1) & 1, abort_flag, p.st, kTimeoutSmemEmpty, (4u << 16) | 14)) break;
        mbar_expect_tx(kv_full, 2 * L::kTile);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_4d(smem + L::kK + c * 16384, &tmK, kv_full, c * 64, t.k0, t.kv_head, t.batch);
          tma_load_4d(smem + L::kV + c * 16384, &tmV, kv_full, c * 64, t.k0, t.kv_head, t.batch);
        }
        for (int it = 0; it < t.iters; ++it, ++g) {
          const int st = g % NS;
          const uint32_t ph = (g / NS) & 1;
          const int head = t.kv_head * group + it / t.per_head;
          const int qi = t.i_min + it % t.per_head;
          if (!mbar_wait(&qdo_empty[st], ph ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (4u << 16) | st)) { ok = false; break; }
          mbar_expect_tx(&qdo_full[st], 2 * L::kTile);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            tma_load_4d(smem + L::kQ + st * L::kTile + c * 16384, &tmQ, &qdo_full[st], c * 64, qi * 128, head, t.batch);
            tma_load_4d(smem + L::kDO + st * L::kTile + c * 16384, &tmDO, &qdo_full[st], c * 64, qi * 128, head, t.batch);
          }
        }
        ++n;
      }
      if (*abort_flag) __nanosleep(50000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(128, 128, 0, 0, 1);
      constexpr uint32_t idesc_acc = make_idesc_f16(128, D, 0, 1, 1);
      const uint32_t sk = smem_u32(smem + L::kK), sv = smem_u32(smem + L::kV);
      const uint32_t spt = smem_u32(smem + L::kPT), sdst = smem_u32(smem + L::kDST);
      int n = 0, g0 = 0;
      bool ok = true;
      // S^T and dP^T of global block g; within a unit they are issued one block ahead (two Q / dO stages), as soon as
      // the element-wise warps hold the previous block's scores in registers
      auto issue_scores = [&](int g) -> bool {
        const int st = g % NS;
        const uint32_t ph = (g / NS) & 1;
        if (!mbar_wait(&qdo_full[st], ph, abort_flag, p.st, kTimeoutSmemFull, (4u << 16) | st)) return false;
        if (g > 0 && !mbar_wait(sdp_taken, (g - 1) & 1, abort_flag, p.st, kTimeoutTmemEmpty, (4u << 16) | 13)) return false;
        tc_fence_after();
        const uint32_t sq = smem_u32(smem + L::kQ + st * L::kTile), sdo = smem_u32(smem + L::kDO + st * L::kTile);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc_mma_f16_ss(tmem_ST, kmajor_desc(sk, kk), kmajor_desc(sq, kk), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          tc_mma_f16_ss(tmem_dPT, kmajor_desc(sv, kk), kmajor_desc(sdo, kk), idesc_s, kk > 0 ? 1u : 0u);
        tc_commit(sdp_full);
        return true;
      };
      constexpr bool kAhead = NS >= 2;
      for (int round = 0; round < snake_rounds(units) && ok; ++round) {
        const int u = snake_unit(round, units);
        if (u < 0) continue;
        const KvUnit t = kv_unit<MODES>(p, u, off, nq);
        if (t.iters == 0) continue;
        if (!mbar_wait(kv_full, n & 1, abort_flag, p.st, kTimeoutSmemFull, (4u << 16) | 8)) break;
        if (kAhead) {
          ok = issue_scores(g0);
          if (ok && t.iters == 1) tc_commit(kv_free);
        }
        for (int it = 0; it < t.iters && ok; ++it) {
          const int g = g0 + it;
          const int st = g % NS;
          if (kAhead) {
            if (it + 1 < t.iters) {
              if (!issue_scores(g + 1)) { ok = false; break; }
              if (it + 2 == t.iters) tc_commit(kv_free);       // the unit's last score products are on their way
            }
          } else {
            if (!issue_scores(g)) { ok = false; break; }
            if (it + 1 == t.iters) tc_commit(kv_free);
          }
          if (!mbar_wait(pds_ready, g & 1, abort_flag, p.st, kTimeoutGeneric, (4u << 16) | 9)) { ok = false; break; }
          if (it == 0 && n > 0) {
            // dV and dK of the previous unit must have been read out before this unit starts its own sums
            if (!mbar_wait(acc_free, (n - 1) & 1, abort_flag, p.st, kTimeoutTmemEmpty, (4u << 16) | 15)) { ok = false; break; }
          }
          tc_fence_after();
          const uint32_t sq = smem_u32(smem + L::kQ + st * L::kTile), sdo = smem_u32(smem + L::kDO + st * L::kTile);
          const int pb = g % PB;
          const uint32_t spt_b = spt + pb * 32768, sdst_b = sdst + pb * 32768;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            tc_mma_f16_ss(tmem_dV, kmajor_desc(spt_b, kk), mnmajor_desc(sdo, kk), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            tc_mma_f16_ss(tmem_dK, kmajor_desc(sdst_b, kk), mnmajor_desc(sq, kk), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&qdo_empty[st]);
          tc_commit(&acc_done[pb]);
        }
        g0 += t.iters;
        ++n;
      }
    }
  } else {
    // Two threads per key row: warps 2..5 take query columns [0, 64) of the block, warps 6..9 columns [64, 128). The
    // columns are independent here (the row statistics come from the forward pass), so the halves never talk.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;       // key row within the block
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    bool ok = true;
    const bool capped = MODES && p.softcap > 0.f;
    const bool special = bounded || capped;
    const float cap_in = capped ? p.scale / p.softcap : 0.f;
    const float cap_l2 = p.softcap * kLog2e;
    int n = 0, g0 = 0;
    // A thread whose wait gave up keeps walking units and blocks without touching tensor memory: the block-wide barrier
    // of the element-wise warps has no time limit of its own, so nobody may leave early.
    for (int round = 0; round < snake_rounds(units); ++round) {
      const int u = snake_unit(round, units);
      if (u < 0) continue;
      const KvUnit t = kv_unit<MODES>(p, u, off, nq);
      const int key = t.k0 + r;
      if (t.iters > 0) {
        auto load_stats = [&](int it, float& l2, float& dl, int& lo) {
          const int head = t.kv_head * group + it / t.per_head;
          const int qr = (t.i_min + it % t.per_head) * 128 + r;
          l2 = INFINITY;
          dl = 0.f;
          if (qr < p.Sq) {
            const size_t idx = (size_t(t.batch) * p.H + head) * p.Sq + qr;
            const float l = p.lse[idx];
            l2 = (l == -INFINITY) ? INFINITY : l * kLog2e;
            dl = p.delta[idx];
          }
          lo = bounded ? flash_row_lo(p, t.batch, qr, off) : 0;
        };
        auto store_stats = [&](float l2, float dl, int lo) {
          s_lse2[r] = l2;
          s_delta[r] = dl;
          s_lo[r] = lo;
        };
        // the previous unit's last block ended with a barrier after its statistics were last read
        if (half == 0) {
          float l2, dl;
          int lo;
          load_stats(0, l2, dl, lo);
          store_stats(l2, dl, lo);
        }
        softmax_bar_sync();
        for (int it = 0; it < t.iters; ++it) {
          const int g = g0 + it;
          const int qrow0 = (t.i_min + it % t.per_head) * 128;
          const int pb = g % PB;
          uint8_t* sPT = smem + L::kPT + pb * 32768;
          uint8_t* sDST = smem + L::kDST + pb * 32768;
          // the statistics of this query block were staged at the end of the previous block; those of the next are
          // fetched now and stored at the end of this one, so their latency hides behind this block's arithmetic
          float n_l2 = INFINITY, n_dl = 0.f;
          int n_lo = 0;
          if (half == 0 && it + 1 < t.iters) load_stats(it + 1, n_l2, n_dl, n_lo);
          if (ok && !mbar_wait(sdp_full, g & 1, abort_flag, p.st, kTimeoutTmemFull, (4u << 16) | 10)) ok = false;
          tc_fence_after();
          // query q (column) sees this key iff key <= q + off  <=>  q >= key - off
          const int first_q = p.causal ? (key - off - qrow0) : 0;    // columns below this are masked
          // this thread's 64 columns: four loads in flight and one wait; the MMA warp may rewrite S^T and dP^T once
          // every thread holds its part in registers
          uint32_t s[2][32], dp[2][32];
          if (ok) {
            tmem_ld_32x32b_x32(tmem_ST + lane_addr + half * 64, s[0]);
            tmem_ld_32x32b_x32(tmem_ST + lane_addr + half * 64 + 32, s[1]);
            tmem_ld_32x32b_x32(tmem_dPT + lane_addr + half * 64, dp[0]);
            tmem_ld_32x32b_x32(tmem_dPT + lane_addr + half * 64 + 32, dp[1]);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(sdp_taken);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) s[0][i] = s[1][i] = dp[0][i] = dp[1][i] = 0u;
          }
          if (ok && g >= PB) {
            // the accumulation that last read this P^T / dS^T buffer (block g - PB) must be complete
            const uint32_t use = uint32_t(g / PB) - 1u;
            if (!mbar_wait(&acc_done[pb], use & 1u, abort_flag, p.st, kTimeoutTmemFull, (4u << 16) | 11)) ok = false;
          }
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int c = half * 2 + cc;
            float pt[32], dst[32];
            if (!special) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int col = c * 32 + i;
                float pr = fast_exp2(__uint_as_float(s[cc][i]) * p.scale_log2 - s_lse2[col]);
                if (col < first_q) pr = 0.f;
                pt[i] = pr;
                dst[i] = pr * (__uint_as_float(dp[cc][i]) - s_delta[col]) * p.scale;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int col = c * 32 + i;
                float sc = __uint_as_float(s[cc][i]), gr = p.scale;
                if (capped) {
                  const float th = tanh_fast(sc * cap_in);
                  sc = th * cap_l2;
                  gr *= 1.f - th * th;
                } else {
                  sc *= p.scale_log2;
                }
                float pr = fast_exp2(sc - s_lse2[col]);
                if (col < first_q || key < s_lo[col]) pr = 0.f;
                pt[i] = pr;
                dst[i] = pr * (__uint_as_float(dp[cc][i]) - s_delta[col]) * gr;
              }
            }
            if (ok) {
              store_operand_chunk(sPT, r, c, pt);
              store_operand_chunk(sDST, r, c, dst);
            }
          }
          if (ok) {
            fence_proxy_async_smem();
            tc_fence_before();
            mbar_arrive(pds_ready);
          }
          softmax_bar_sync();    // this block's statistics are no longer read
          if (half == 0 && it + 1 < t.iters) store_stats(n_l2, n_dl, n_lo);
          softmax_bar_sync();    // the next block's are visible
        }
        if (ok) {
          const int last = g0 + t.iters - 1;
          if (!mbar_wait(&acc_done[last % PB], uint32_t(last / PB) & 1u, abort_flag, p.st, kTimeoutTmemFull, (4u << 16) | 12))
            ok = false;
        }
        tc_fence_after();
      }
      // write-out: the first half of the threads takes dV, the second dK; the sums leave tensor memory first so that the
      // next unit may start accumulating while the rows are packed and stored
      uint32_t o[D];
      if (t.iters > 0 && ok) {
        const uint32_t acc = half ? tmem_dK : tmem_dV;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld_32x32b_x32(acc + lane_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&o[c * 32]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(acc_free);
      } else {
#pragma unroll
        for (int i = 0; i < D; ++i) o[i] = 0u;
      }
      if ((ok || t.iters == 0) && key < p.Skv) {
        __nv_bfloat16* drow = (half ? p.dK + (size_t(t.batch) * p.Skv + key) * p.dk_row_stride
                                    : p.dV + (size_t(t.batch) * p.Skv + key) * p.dv_row_stride) + size_t(t.kv_head) * D;
#pragma unroll
        for (int gq = 0; gq < D / 8; ++gq) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[gq * 8 + 0]), __uint_as_float(o[gq * 8 + 1]));
          w.y = pack_bf16x2(__uint_as_float(o[gq * 8 + 2]), __uint_as_float(o[gq * 8 + 3]));
          w.z = pack_bf16x2(__uint_as_float(o[gq * 8 + 4]), __uint_as_float(o[gq * 8 + 5]));
          w.w = pack_bf16x2(__uint_as_float(o[gq * 8 + 6]), __uint_as_float(o[gq * 8 + 7]));
          *reinterpret_cast<uint4*>(drow + gq * 8) = w;
        }
      }
      if (t.iters > 0) {
        g0 += t.iters;
        ++n;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D, bool MODES>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const FlashParams& p, cudaStream_t stream) {
  auto kq = flash_bwd_q_kernel<D, MODES>;
  auto kkv = flash_bwd_kv_kernel<D, MODES>;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        cudaError_t e1 = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdQSmem<D>::kTotal);
        if (e1 != cudaSuccess) return int(e1);
        return int(cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdKVSmem<D>::kTotal));
      }))
    return e;
  const int q_units = ((p.Sq + 127) / 128) * p.H * p.B;
  kq<<<min(q_units, sm_count()), kBwdThreads, BwdQSmem<D>::kTotal, stream>>>(tq, tk, tv, tdo, p);
  note_launches(1);
  int rc = int(cudaGetLastError());
  if (rc) return rc;
  const int kv_units = ((p.Skv + 127) / 128) * p.Hkv * p.B;
  kkv<<<min(kv_units, sm_count()), kBwdThreads, BwdKVSmem<D>::kTotal, stream>>>(tq, tk, tv, tdo, p);
  note_launches(1);
  return int(cudaGetLastError());
}

}  // namespace idrak

using namespace idrak;

// out / dout: contiguous [B, Sq, H, D]; lse, delta [B,H,Sq]. dq / dk / dv rows hold heads packed [heads, D] with
// the given row strides in elements (0 = contiguous), so they may be slices of one fused d(QKV) buffer;
// their batch stride is rows * row stride.
// window > 0 and row_start (one int per query row, [B, Sq]) restrict the keys a query sees exactly as in the forward
// entry point; both need `causal`. `softcap` > 0 differentiates through the tanh cap of the forward.
IDRAK_API int idrak_flash_bwd_ex(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                 const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int H, int Hkv,
                                 int Sq, int Skv, int D, long long q_row_stride, long long k_row_stride,
                                 long long v_row_stride, long long q_batch_stride, long long k_batch_stride,
                                 long long v_batch_stride, long long dq_row_stride, long long dk_row_stride,
                                 long long dv_row_stride, float scale, int causal, int window, const int* row_start,
                                 float softcap, void* stream_) {
  if (D != 64 && D != 128) return -2;
  if (H % Hkv) return -3;
  if ((window > 0 || row_start) && !causal) return -4;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  {
    const long long rows = (long long)B * Sq * H;
    const int threads = 256;
    const long long blocks = (rows * (D / 8) + threads - 1) / threads;
    flash_delta_kernel<<<unsigned(blocks), threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(out),
                                                                 static_cast<const __nv_bfloat16*>(dout), delta, B,
                                                                 Sq, H, D);
    note_launches(1);
    int rc = int(cudaGetLastError());
    if (rc) return rc;
  }
  FlashParams p;
  p.O = nullptr;
  p.o_row_stride = 0;
  p.lse = const_cast<float*>(lse);
  p.delta = delta;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.causal = causal;
  p.window = window > 0 ? window : 0;
  p.row_start = row_start;
  p.softcap = softcap > 0.f ? softcap : 0.f;
  p.st = status_device_ptr();
  p.dQ = static_cast<__nv_bfloat16*>(dq);
  p.dK = static_cast<__nv_bfloat16*>(dk);
  p.dV = static_cast<__nv_bfloat16*>(dv);
  p.dq_row_stride = dq_row_stride > 0 ? dq_row_stride : (long long)H * D;
  p.dk_row_stride = dk_row_stride > 0 ? dk_row_stride : (long long)Hkv * D;
  p.dv_row_stride = dv_row_stride > 0 ? dv_row_stride : (long long)Hkv * D;
  CUtensorMap tq, tk, tv, tdo;
  if (make_head_map(&tq, q, D, Sq, H, B, q_row_stride, q_batch_stride)) return -10;
  if (make_head_map(&tk, k, D, Skv, Hkv, B, k_row_stride, k_batch_stride)) return -11;
  if (make_head_map(&tv, v, D, Skv, Hkv, B, v_row_stride, v_batch_stride)) return -12;
  if (make_head_map(&tdo, dout, D, Sq, H, B, (long long)H * D, (long long)Sq * H * D)) return -13;
  if (p.window > 0 || p.row_start || p.softcap > 0.f)
    return D == 64 ? launch_bwd<64, true>(tq, tk, tv, tdo, p, stream) : launch_bwd<128, true>(tq, tk, tv, tdo, p, stream);
  return D == 64 ? launch_bwd<64, false>(tq, tk, tv, tdo, p, stream) : launch_bwd<128, false>(tq, tk, tv, tdo, p, stream);
}

IDRAK_API int idrak_flash_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                              const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int H, int Hkv,
                              int Sq, int Skv, int D, long long q_row_stride, long long k_row_stride,
                              long long v_row_stride, long long q_batch_stride, long long k_batch_stride,
                              long long v_batch_stride, long long dq_row_stride, long long dk_row_stride,
                              long long dv_row_stride, float scale, int causal, void* stream_) {
  return idrak_flash_bwd_ex(q, k, v, out, dout, lse, delta, dq, dk, dv, B, H, Hkv, Sq, Skv, D, q_row_stride,
                            k_row_stride, v_row_stride, q_batch_stride, k_batch_stride, v_batch_stride, dq_row_stride,
                            dk_row_stride, dv_row_stride, scale, causal, 0, nullptr, 0.f, stream_);
}
