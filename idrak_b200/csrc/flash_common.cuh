// Shared by the flash-attention forward and backward kernels.
#pragma once
#include "common.cuh"

namespace idrak {

struct FlashParams {
  __nv_bfloat16* O;
  long long o_row_stride;
  float* lse;          // [B, H, Sq]
  int B, H, Hkv, Sq, Skv;
  float scale, scale_log2;
  int causal;
  // Optional lower bounds on the keys a query may see (both need `causal`):
  //   window     > 0: query at position r sees keys (r + off - window, r + off] only (sliding-window attention)
  //   row_start  per query row [B * Sq]: the first key index it may see - the start of its own sequence when several
  //              sequences are packed into one row of the batch. Must not decrease along a row of the batch.
  int window;
  const int* row_start;
  // logit soft-capping: scores become softcap * tanh(scale * s / softcap) before the softmax (0 = off; forward only)
  float softcap;
  Status* st;
  // backward only
  const float* delta;  // [B, H, Sq] rowsum(dO * O)
  __nv_bfloat16* dQ;
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  long long dq_row_stride, dk_row_stride, dv_row_stride;
};

// 2^x as one MUFU instruction (flush-to-zero, about 2 ulp): the softmax exponentials are the bulk of the element-wise
// work and the library routine spends several instructions per call on range handling the scores do not need
// (-inf gives 0, large negative arguments flush to 0).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Barrier `id` (1..15) over `threads` threads of the CTA (whole warps).
__device__ __forceinline__ void flash_bar_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// First key index query `row` (position in its batch entry) may see; off = Skv - Sq.
__device__ __forceinline__ int flash_row_lo(const FlashParams& p, int batch, int row, int off) {
  int lo = 0;
  if (p.window > 0) lo = max(lo, row + off - p.window + 1);
  if (p.row_start && row < p.Sq) lo = max(lo, p.row_start[size_t(batch) * p.Sq + row]);
  return lo;
}

// 4-D map (d, position, head, batch) over a buffer whose rows hold heads packed as [heads, D].
// Box = 64 d x 128 positions: one 128-byte-swizzled operand tile column block.
static inline int make_head_map(CUtensorMap* tm, const void* ptr, int D, int S, int heads, int B,
                                long long row_stride, long long batch_stride) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(S), uint64_t(heads), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(row_stride) * 2, uint64_t(D) * 2, uint64_t(batch_stride) * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return encode_tensor_map(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace idrak
