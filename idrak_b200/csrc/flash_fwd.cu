// Flash attention forward for sm_100a (prefill / training): O = softmax(scale * Q K^T + mask) V without
// ever forming the score matrix in memory. Causal or full, grouped-query heads, head size 64 or 128.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key/value sequence in blocks of 128:
//   warp 0      TMA producer: Q once, then K and V blocks through two-stage rings (128B swizzle)
//   warp 1      MMA issuer:   S = Q K^T into one of TWO score buffers in TMEM (tcgen05.mma, K-major x K-major), issued
//                             one block ahead so the scores of block j+1 are being computed while block j is in the
//                             softmax; then O += P V (P from shared memory, V as an MN-major operand, accumulator in TMEM)
//   warps 2..9  softmax:      two threads per query row, each with 64 of the block's 128 score columns in registers
//                             (two tcgen05.ld in flight, one wait); the score buffer goes back to the MMA warp at
//                             once; the halves exchange row maxima through shared memory, take the online max /
//                             sum in the log2 domain, write P as bf16 into the swizzled operand layout, rescale
//                             their half of the TMEM accumulator only when the running max moved by more than 2^8
//                             (warp-uniform decision), and finally normalise and store O plus the row
//                             log-sum-exp for the backward pass. Eight softmax warps per CTA, two CTAs per SM at
//                             head size 64: four warps per scheduler to hide the latencies of the chain.
// Q, K and V are addressed through 4-D tensor maps (d, position, head, batch) so fused-QKV buffers and
// cache layouts need no copy.
//
// Reference counterparts: flash_tc_fwd_d{64,128} (src/Idrak.Gpu/Cuda/PtxKernels.FlashTensorCore.cs:318-321)
// and Tensor.CausalAttention (src/Idrak.Abstraction/Tensors/Tensor.Decoding.cs:132).
#include "flash_common.cuh"

namespace idrak {

template <int D>
struct FwdSmem {
  static constexpr int kTile = 128 * D * 2;        // one 128-row operand tile
  static constexpr int kP = 128 * 128 * 2;
  static constexpr int kQ = 0;
  // Head size 64 keeps ONE key stage: Q K^T of a block finishes before that block's softmax starts, so the next keys
  // load during the softmax anyway, and the 16 KB saved are what lets two CTAs share an SM (2 x 100 KB): with one CTA
  // per SM its set-up and write-out (about 6 us) ran unhidden, half of the time at 1024 tokens.
  static constexpr int kKStages = (D == 64) ? 1 : 2;
  static constexpr int kK = kQ + kTile;
  static constexpr int kV = kK + kKStages * kTile;  // two stages
  static constexpr int kPOff = kV + 2 * kTile;
  static constexpr int kXch = kPOff + kP;          // row maxima / sums exchanged between the two halves: 2 x 2 x 128 floats
  static constexpr int kBar = kXch + 2048;
  static constexpr int kTotal = kBar + 256 + 1024;
};

constexpr int kFwdThreads = 320;   // TMA warp, MMA warp, eight softmax warps

// MODES = false compiles the window / packed-sequence / soft-cap code out: the plain causal kernel is unchanged by them
template <int D, bool MODES>
__global__ void __launch_bounds__(kFwdThreads, (D == 64) ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  using L = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* k_empty = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_empty = bars + 11;  // [2]
  uint64_t* p_ready = bars + 13;
  uint64_t* o_done = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavier (later) causal row blocks are scheduled first
  const int qb = p.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.H / p.Hkv);
  const int q0 = qb * 128;
  const int off = p.Skv - p.Sq;   // causal: query row r sees keys <= r + off
  int nkv_end = (p.Skv + 127) / 128;
  if (p.causal) nkv_end = min(nkv_end, (q0 + 127 + off) / 128 + 1);
  if (nkv_end < 0) nkv_end = 0;
  // key blocks wholly below what the tile's first row may see are skipped (the bounds do not decrease along rows)
  const bool bounded = MODES && p.causal && (p.window > 0 || p.row_start != nullptr);
  const int jlo = bounded ? min(nkv_end, max(0, flash_row_lo(p, batch, min(q0, p.Sq - 1), off)) / 128) : 0;
  const int nkv = nkv_end - jlo;      // blocks this CTA walks: key block of iteration j is jlo + j

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], 256);
    }
    mbar_init(p_ready, 256);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    if (nkv > 0) {
      // The first loads go out before the CTA-wide sync below (this thread is also the producer): their latency
      // overlaps the tensor-memory allocation instead of following it.
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, L::kTile);
      mbar_expect_tx(&k_full[0], L::kTile);
      mbar_expect_tx(&v_full[0], L::kTile);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_4d(smem + L::kQ + c * 16384, &tmQ, q_full, c * 64, q0, head, batch);
        tma_load_4d(smem + L::kK + c * 16384, &tmK, &k_full[0], c * 64, jlo * 128, kv_head, batch);
        tma_load_4d(smem + L::kV + c * 16384, &tmV, &v_full[0], c * 64, jlo * 128, kv_head, batch);
      }
    }
  }
  // D = 64: one score buffer [0,128) and O at [128,192) in 256 columns, so two CTAs share an SM (one CTA's prologue and
  // epilogue hide behind the other's main loop); the buffer is handed back as soon as the row sits in registers, which
  // lets the next block's scores be computed during this block's softmax all the same.
  // D = 128: two score buffers at [0,128) and [128,256), O at [256,384), one CTA per SM.
  constexpr int kSBufs = (D == 64) ? 1 : 2;
  constexpr uint32_t kTmemCols = (D == 64) ? 256 : 512;
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128 * kSBufs;

  if (warp == 0) {
    if (lane == 0 && nkv > 0) {
      uint32_t inflight = 0;
      bool ok = true;
      for (int j = 1; j < nkv && ok; ++j) {          // block 0 was requested before the sync
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kst = (L::kKStages == 2) ? st : 0;
        const uint32_t kph = (L::kKStages == 2) ? ph : uint32_t(j & 1);
        if (!mbar_wait(&k_empty[kst], kph ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (2u << 16) | kst)) { ok = false; break; }
        mbar_expect_tx(&k_full[kst], L::kTile);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + L::kK + kst * L::kTile + c * 16384, &tmK, &k_full[kst], c * 64, (jlo + j) * 128, kv_head, batch);
        inflight |= 1u << st;
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.st, kTimeoutSmemEmpty, (2u << 16) | (2 + st))) { ok = false; break; }
        mbar_expect_tx(&v_full[st], L::kTile);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(smem + L::kV + st * L::kTile + c * 16384, &tmV, &v_full[st], c * 64, (jlo + j) * 128, kv_head, batch);
        inflight |= 4u << st;
      }
      if (!ok || *abort_flag) {
        // let copies already issued land before shared memory is released (bounded)
        for (int i = 0; i < (1 << 16); ++i) {
          if (!mbar_try_wait(q_full, 0)) continue;
          break;
        }
        __nanosleep(20000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nkv > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(128, 128, 0, 0, 1);
      constexpr uint32_t idesc_o = make_idesc_f16(128, D, 0, 1, 1);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.st, kTimeoutSmemFull, (2u << 16) | 8);
      const uint32_t sq = smem_u32(smem + L::kQ);
      const uint32_t sp = smem_u32(smem + L::kPOff);
      // scores of block j go to buffer j & 1; they are issued one block ahead of the P V product
      auto issue_scores = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kst = (L::kKStages == 2) ? st : 0;
        const uint32_t kph = (L::kKStages == 2) ? ph : uint32_t(j & 1);
        if (!mbar_wait(&k_full[kst], kph, abort_flag, p.st, kTimeoutSmemFull, (2u << 16) | kst)) return false;
        // the buffer's previous use (block j - 2) has been read out by the softmax warps
        const int sb = (kSBufs == 2) ? st : 0;
        const uint32_t sph = (kSBufs == 2) ? (ph ^ 1) : uint32_t((j + 1) & 1);     // the buffer's previous use: block j - kSBufs
        if (!mbar_wait(&s_empty[sb], sph, abort_flag, p.st, kTimeoutTmemEmpty, (2u << 16) | (12 + sb))) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + L::kK + kst * L::kTile);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t o = (kk >> 2) * 16384 + (kk & 3) * 32;
          tc_mma_f16_ss(tmem_S + sb * 128, make_smem_desc_sw128(sq + o, 16, 1024), make_smem_desc_sw128(sk + o, 16, 1024),
                        idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[sb]);
        tc_commit(&k_empty[kst]);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < nkv && !issue_scores(j + 1)) { ok = false; break; }
        if (!mbar_wait(p_ready, j & 1, abort_flag, p.st, kTimeoutGeneric, (2u << 16) | 9)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], ph, abort_flag, p.st, kTimeoutSmemFull, (2u << 16) | (2 + st))) { ok = false; break; }
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + L::kV + st * L::kTile);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t da = make_smem_desc_sw128(sp + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sv + kk * 2048, 16384, 1024);
          tc_mma_f16_ss(tmem_O, da, db, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&v_empty[st]);
        tc_commit(o_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    // Two threads per query row: warps 2..5 take key columns [0, 64) of a block, warps 6..9 columns [64, 128); the
    // two warps that share a TMEM lane quarter (w and w + 4) own the same 32 rows. Eight softmax warps per CTA (and two
    // CTAs per SM at head size 64) give every scheduler four of them to switch between while one waits on a load,
    // the exponential unit or a barrier. The halves exchange their row maxima through shared memory once per block
    // (slots alternate with the block's parity) and their row sums once at the end.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;            // which 64 columns of the block
    const int r = quarter * 32 + lane;           // row within the tile == TMEM lane
    const int row = q0 + r;                      // query position
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    uint8_t* sP = smem + L::kPOff;
    float* xch = reinterpret_cast<float*>(smem + L::kXch);      // [2 parities][2 halves][128 rows]
    const uint32_t pair_bar = 1 + quarter;       // named barrier of the two warps of this lane quarter
    float m_used = -INFINITY;                    // max the accumulator and the running sum are scaled by
    float l = 0.f;                               // this thread's part of the row sum
    bool ok = nkv > 0;
    const int row_lo = bounded ? flash_row_lo(p, batch, row, off) : 0;     // first key this row may see
    const bool capped = MODES && p.softcap > 0.f;
    const float cap_in = capped ? p.scale / p.softcap : 0.f;               // s -> softcap * tanh(s * scale / softcap)
    const float sl2 = capped ? p.softcap * 1.4426950408889634f : p.scale_log2;   // factor into the log2 domain
    constexpr int kOC = D / 2;                   // accumulator columns this thread rescales and stores
    // A thread whose wait gave up keeps walking the loop (skipping the waits and the tensor-memory traffic): its partner
    // meets it at the pair's barrier in every block, and that barrier has no time limit of its own.
    for (int j = 0; j < nkv; ++j) {
      const int sb = (kSBufs == 2) ? (j & 1) : 0;
      const uint32_t sph = (kSBufs == 2) ? uint32_t((j >> 1) & 1) : uint32_t(j & 1);
      if (ok && !mbar_wait(&s_full[sb], sph, abort_flag, p.st, kTimeoutTmemFull, (2u << 16) | 10)) ok = false;
      tc_fence_after();
      const int k0 = (jlo + j) * 128 + half * 64;          // first key of this thread's 64 columns
      // keys visible to this row among its 64 columns: [lo, lim)
      int lim = p.Skv - k0;
      if (p.causal) lim = min(lim, row + off - k0 + 1);
      lim = max(0, min(64, lim));
      const int lo = max(0, min(64, row_lo - k0));
      const bool need_mask = lim < 64 || lo > 0;
      uint32_t s[2][32];
      if (ok) {
        const uint32_t s_addr = tmem_S + uint32_t(sb) * 128 + lane_addr + half * 64;
        tmem_ld_32x32b_x32(s_addr + 0, s[0]);
        tmem_ld_32x32b_x32(s_addr + 32, s[1]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&s_empty[sb]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) s[0][i] = s[1][i] = 0u;
      }
      if (capped) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) s[c][i] = __float_as_uint(tanh_fast(__uint_as_float(s[c][i]) * cap_in));
      }
      float m2[2] = {-INFINITY, -INFINITY};
      if (!need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          m2[0] = fmaxf(m2[0], __uint_as_float(s[0][i]));
          m2[1] = fmaxf(m2[1], __uint_as_float(s[1][i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
            if (c * 32 + i < lim && c * 32 + i >= lo) m2[c] = fmaxf(m2[c], __uint_as_float(s[c][i]));
        }
      }
      // the row maximum over both halves (every thread reaches this barrier, whatever `ok` says, so its partner never
      // waits for nothing)
      float* slot = xch + (j & 1) * 256;
      slot[half * 128 + r] = fmaxf(m2[0], m2[1]);
      flash_bar_sync(pair_bar, 64);
      float mx = fmaxf(slot[r], slot[128 + r]);
      mx *= sl2;
      const float m_new = fmaxf(m_used, mx);
      // the accumulator is rescaled only when some row of this warp moved its max by more than 2^8 (both warps of a
      // quarter hold the same rows and so decide alike)
      const bool need = (j > 0) && (m_new - m_used > 8.0f);
      const bool warp_rescale = __any_sync(0xffffffffu, need);
      if (j > 0 && ok) {
        // P of the previous block is still being read by its MMA until o_done completes
        if (!mbar_wait(o_done, (j - 1) & 1, abort_flag, p.st, kTimeoutTmemFull, (2u << 16) | 11)) ok = false;
        tc_fence_after();
      }
      if (j == 0) {
        m_used = m_new;
      } else if (warp_rescale) {
        const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_used - m_new);
        m_used = m_new;
        l *= alpha;
        if (ok) {
#pragma unroll 1
          for (int c = 0; c < kOC / 16; ++c) {          // 16 columns at a time: the 64 scores stay in registers beside them
            uint32_t o[16];
            tmem_ld_32x32b_x16(tmem_O + lane_addr + half * kOC + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x16(tmem_O + lane_addr + half * kOC + c * 16, o);
          }
          tmem_st_wait();
        }
      }
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      // probabilities -> bf16 operand tile (K-major, 128B swizzle: chunk ^= row % 8), from the registers
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
        uint8_t* atom = sP + half * 16384 + r * 128;          // columns [64 half, 64 half + 64) are one 128-byte row
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          // eight exponentials, packed and stored at once: few values live at a time (96 registers per thread)
          float pv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int col = c * 32 + g * 8 + i;
            float e = fast_exp2(__uint_as_float(s[c][g * 8 + i]) * sl2 - m_sub);
            if (need_mask && (col >= lim || col < lo)) e = 0.f;
            pv[i] = e;
            l4[i & 3] += e;
          }
          const int chunk = (c * 4 + g) ^ (r & 7);
          uint4 o;
          o.x = pack_bf16x2(pv[0], pv[1]);
          o.y = pack_bf16x2(pv[2], pv[3]);
          o.z = pack_bf16x2(pv[4], pv[5]);
          o.w = pack_bf16x2(pv[6], pv[7]);
          *reinterpret_cast<uint4*>(atom + chunk * 16) = o;
        }
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      }
      if (ok) {
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(p_ready);
      }
    }
    if (ok && nkv > 0) {
      if (!mbar_wait(o_done, (nkv - 1) & 1, abort_flag, p.st, kTimeoutTmemFull, (2u << 16) | 12)) ok = false;
    }
    tc_fence_after();
    // the row sum over both halves
    float* slot = xch + (nkv & 1) * 256;
    slot[half * 128 + r] = l;
    flash_bar_sync(pair_bar, 64);
    const float l_row = slot[r] + slot[128 + r];
    if (nkv <= 0) {
      // no visible key: output zeros, lse = -inf
      if (row < p.Sq) {
        __nv_bfloat16* orow = p.O + (size_t(batch) * p.Sq + row) * p.o_row_stride + size_t(head) * D + half * kOC;
        for (int i = 0; i < kOC; i += 8) *reinterpret_cast<uint4*>(orow + i) = make_uint4(0, 0, 0, 0);
        if (p.lse && half == 0) p.lse[(size_t(batch) * p.H + head) * p.Sq + row] = -INFINITY;
      }
    } else if (ok) {
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
      __nv_bfloat16* orow = p.O + (size_t(batch) * p.Sq + row) * p.o_row_stride + size_t(head) * D + half * kOC;
#pragma unroll 1
      for (int c = 0; c < kOC / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_O + lane_addr + half * kOC + c * 32, o);
        tmem_ld_wait();
        if (row < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = w;
          }
        }
      }
      if (row < p.Sq && p.lse && half == 0) {
        // natural-log LSE of the scaled scores
        p.lse[(size_t(batch) * p.H + head) * p.Sq + row] =
            (l_row > 0.f) ? (m_used + log2f(l_row)) * 0.6931471805599453f : -INFINITY;
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
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashParams& p,
                      cudaStream_t stream) {
  using L = FwdSmem<D>;
  auto kern = flash_fwd_kernel<D, MODES>;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      }))
    return e;
  dim3 grid((p.Sq + 127) / 128, p.H, p.B);
  kern<<<grid, kFwdThreads, L::kTotal, stream>>>(tq, tk, tv, p);
  note_launches(1);
  return int(cudaGetLastError());
}

}  // namespace idrak

using namespace idrak;

// q: rows of (batch, position) with `q_row_stride` elements between positions and heads packed as
// [H, D] inside a row; likewise k, v with Hkv heads. o: [B*Sq, o_row_stride] with heads packed [H, D].
// lse: [B, H, Sq] fp32 (may be null). Pointers 16-byte aligned, strides multiples of 8 elements.
// `window` > 0 (sliding window), `row_start` ([B * Sq] int32: the first key each query row may see, for sequences packed
// into one batch row) and `softcap` > 0 (tanh soft-capping of the scaled scores) are the optional modes; the first
// two need `causal`. Reference: window and soft-cap of attention_flash_* (src/Idrak.Gpu/Cuda/PtxKernels.Rows.cs:779),
// per-row key ranges of the span kernels (PtxKernels.SpansTiled.cs).
IDRAK_API int idrak_flash_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                                 int Hkv, int Sq, int Skv, int D, long long q_row_stride, long long k_row_stride,
                                 long long v_row_stride, long long o_row_stride, long long q_batch_stride,
                                 long long k_batch_stride, long long v_batch_stride, float scale, int causal,
                                 int window, const int* row_start, float softcap, void* stream_) {
  if (D != 64 && D != 128) return -2;
  if (H % Hkv) return -3;
  if ((window > 0 || row_start) && !causal) return -4;
  FlashParams p;
  p.O = static_cast<__nv_bfloat16*>(o);
  p.o_row_stride = o_row_stride;
  p.lse = lse;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.window = window > 0 ? window : 0;
  p.row_start = row_start;
  p.softcap = softcap > 0.f ? softcap : 0.f;
  p.st = status_device_ptr();
  CUtensorMap tq, tk, tv;
  if (make_head_map(&tq, q, D, Sq, H, B, q_row_stride, q_batch_stride)) return -10;
  if (make_head_map(&tk, k, D, Skv, Hkv, B, k_row_stride, k_batch_stride)) return -11;
  if (make_head_map(&tv, v, D, Skv, Hkv, B, v_row_stride, v_batch_stride)) return -12;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (p.window > 0 || p.row_start || p.softcap > 0.f)
    return D == 64 ? launch_fwd<64, true>(tq, tk, tv, p, stream) : launch_fwd<128, true>(tq, tk, tv, p, stream);
  return D == 64 ? launch_fwd<64, false>(tq, tk, tv, p, stream) : launch_fwd<128, false>(tq, tk, tv, p, stream);
}

IDRAK_API int idrak_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                              int Hkv, int Sq, int Skv, int D, long long q_row_stride, long long k_row_stride,
                              long long v_row_stride, long long o_row_stride, long long q_batch_stride,
                              long long k_batch_stride, long long v_batch_stride, float scale, int causal,
                              void* stream_) {
  return idrak_flash_fwd_ex(q, k, v, o, lse, B, H, Hkv, Sq, Skv, D, q_row_stride, k_row_stride, v_row_stride,
                            o_row_stride, q_batch_stride, k_batch_stride, v_batch_stride, scale, causal, 0, nullptr, 0.f,
                            stream_);
}
