// Fused softmax cross-entropy as a bulk-copy pipeline: rows of up to 57,344 logits (112 KB of bf16).
//
// The register kernel (xent.cu) gives a row to a 1024-thread block that loads it, reduces twice and stores the
// gradient; nothing overlaps the load of the next row with the arithmetic and the store of this one, and it sits
// near a third of HBM speed. Here one persistent CTA per SM keeps two rows in shared memory: a producer thread
// streams row i + 1 in with one cp.async.bulk while sixteen consumer warps work on row i in place - maximum, sum of
// exponentials, gradient - and the finished row leaves with one bulk store, so loads, arithmetic and stores of
// neighbouring rows run at the same time. Each exponential is evaluated once: the second pass leaves exp(x - max)
// in the row (bf16) and the third scales it.
//
// Same contract as idrak_softmax_xent: loss per row, optional log-sum-exp, logits overwritten by
// (softmax - onehot) * scale, padding columns (vocab <= c < ld) get 0, ignored rows get loss 0 and gradient 0.
// Every wait is bounded and reports through the status word.
//
// Reference counterpart: softmax_ce_rows_f32 (src/Idrak.Gpu/Cuda/PtxKernels.Decoder.cs:12,75-77).
#include "common.cuh"
#include <cstdlib>

namespace idrak {

constexpr int kXbConsumers = 512;
constexpr int kXbThreads = kXbConsumers + 32;
constexpr int kXbMaxRowBytes = 112 * 1024;

__device__ __forceinline__ void xb_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void xb_bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(gdst)),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kXbConsumers) : "memory"); }
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Reduce over the 16 consumer warps; every consumer thread gets the result, summed / maxed in warp order.
__device__ __forceinline__ float consumer_reduce(float v, float* sm, bool is_max) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  consumer_sync();
  if (lane == 0) sm[wid] = v;
  consumer_sync();
  float r = sm[0];
#pragma unroll
  for (int i = 1; i < kXbConsumers / 32; ++i) r = is_max ? fmaxf(r, sm[i]) : r + sm[i];
  return r;
}

struct XentBulkParams {
  __nv_bfloat16* logits;
  const int* targets;
  float* losses;
  float* lse_out;
  int rows, vocab, ld;
  float scale;
  int ignore_index, write_grad;
  Status* st;
};

__global__ void __launch_bounds__(kXbThreads, 1) xent_bulk_kernel(const XentBulkParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const uint32_t row_bytes = uint32_t(p.ld) * 2;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + 2 * size_t(row_bytes));
  uint64_t* done = full + 2;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(done + 2);
  float* red = reinterpret_cast<float*>(done + 3);          // 16 floats

  const int my_rows = (p.rows - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();

  if (threadIdx.x >= kXbConsumers) {
    // ------------------------------------------------------------------ producer (one thread): loads and stores
    if (threadIdx.x == kXbConsumers) {
      bool ok = true;
      uint32_t issued_mask = 0, issued_phase = 0;
      for (int i = 0; i < my_rows && ok; ++i) {
        const int stage = i & 1;
        const uint32_t phase = (i >> 1) & 1;
        // the row that last used this stage has been stored out of it
        if (p.write_grad) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        const size_t row = size_t(blockIdx.x) + size_t(i) * gridDim.x;
        mbar_expect_tx(&full[stage], row_bytes);
        xb_bulk_load(smem + size_t(stage) * row_bytes, p.logits + row * p.ld, row_bytes, &full[stage]);
        issued_mask |= 1u << stage;
        issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
        if (i >= 1) {
          const int ps = (i - 1) & 1;
          if (!mbar_wait(&done[ps], ((i - 1) >> 1) & 1, abort_flag, p.st, kTimeoutGeneric, (10u << 16) | ps)) {
            ok = false;
            break;
          }
          if (p.write_grad) {
            const size_t prow = size_t(blockIdx.x) + size_t(i - 1) * gridDim.x;
            xb_bulk_store(p.logits + prow * p.ld, smem + size_t(ps) * row_bytes, row_bytes);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      }
      if (ok && my_rows > 0) {
        const int i = my_rows - 1, ps = i & 1;
        if (mbar_wait(&done[ps], (i >> 1) & 1, abort_flag, p.st, kTimeoutGeneric, (10u << 16) | ps) && p.write_grad) {
          const size_t prow = size_t(blockIdx.x) + size_t(i) * gridDim.x;
          xb_bulk_store(p.logits + prow * p.ld, smem + size_t(ps) * row_bytes, row_bytes);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (*abort_flag) {
        // give up: let the loads already issued land before the CTA's shared memory goes away
        for (int s = 0; s < 2; ++s) {
          if (issued_mask & (1u << s)) {
            const uint32_t par = (issued_phase >> s) & 1u;
            for (int k = 0; k < (1 << 20); ++k)
              if (mbar_try_wait(&full[s], par)) break;
          }
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // stores complete before shared memory goes away
    }
    return;
  }

  // -------------------------------------------------------------------- consumers: one row at a time, in place
  const int nvec = p.ld >> 3;
  const float l2e = 1.4426950408889634f;
  for (int i = 0; i < my_rows; ++i) {
    const int stage = i & 1;
    if (!mbar_wait(&full[stage], (i >> 1) & 1, abort_flag, p.st, kTimeoutSmemFull, (10u << 16) | stage)) break;
    const int row = int(blockIdx.x) + i * int(gridDim.x);
    uint4* srow = reinterpret_cast<uint4*>(smem + size_t(stage) * row_bytes);
    const int target = p.targets[row];
    const bool ignored = (target == p.ignore_index) || target < 0 || target >= p.vocab;
    float target_logit = 0.f;
    if (threadIdx.x == 0 && !ignored)
      target_logit = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(srow)[target]);
    float mx = -INFINITY;
    for (int vi = threadIdx.x; vi < nvec; vi += kXbConsumers) {
      const uint4 r = srow[vi];
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
      const int c0 = vi * 8;
      if (c0 + 8 <= p.vocab) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16x2(w[k]);
          mx = fmaxf(mx, fmaxf(f.x, f.y));
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16x2(w[k]);
          if (c0 + 2 * k < p.vocab) mx = fmaxf(mx, f.x);
          if (c0 + 2 * k + 1 < p.vocab) mx = fmaxf(mx, f.y);
        }
      }
    }
    mx = consumer_reduce(mx, red, true);        // (its barriers also order the read of the target logit before pass 2)
    const float shift = -mx * l2e;
    float se = 0.f;
    for (int vi = threadIdx.x; vi < nvec; vi += kXbConsumers) {
      const uint4 r = srow[vi];
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
      uint32_t o[4];
      const int c0 = vi * 8;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16x2(w[k]);
        float e0 = ex2_fast(fmaf(f.x, l2e, shift));
        float e1 = ex2_fast(fmaf(f.y, l2e, shift));
        if (c0 + 8 > p.vocab) {
          if (c0 + 2 * k >= p.vocab) e0 = 0.f;
          if (c0 + 2 * k + 1 >= p.vocab) e1 = 0.f;
        }
        se += e0 + e1;
        o[k] = pack_bf16x2(e0, e1);
      }
      if (p.write_grad) srow[vi] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    se = consumer_reduce(se, red, false);
    if (threadIdx.x == 0) {
      const float lse = mx + logf(se);
      p.losses[row] = ignored ? 0.f : (lse - target_logit);
      if (p.lse_out) p.lse_out[row] = lse;
    }
    if (p.write_grad) {
      const float inv = ignored ? 0.f : p.scale / se;
      for (int vi = threadIdx.x; vi < nvec; vi += kXbConsumers) {
        const uint4 r = srow[vi];
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
        uint32_t o[4];
        const int c0 = vi * 8;
        const bool has_target = !ignored && target >= c0 && target < c0 + 8;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16x2(w[k]);
          float g0 = f.x * inv, g1 = f.y * inv;
          if (has_target) {
            if (c0 + 2 * k == target) g0 -= p.scale;
            if (c0 + 2 * k + 1 == target) g1 -= p.scale;
          }
          o[k] = pack_bf16x2(g0, g1);
        }
        srow[vi] = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_proxy_async_smem();      // the bulk store reads what these threads wrote
    }
    consumer_sync();
    if (threadIdx.x == 0) mbar_arrive(&done[stage]);
  }
}

// Returns -100 when the sizes do not fit this kernel (the caller then takes the register kernels).
int xent_bulk_launch(void* logits, const int* targets, float* losses, float* lse, int rows, int vocab, int ld,
                     float scale, int ignore_index, int write_grad, cudaStream_t stream) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("IDRAK_XENT_BULK");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  const size_t row_bytes = size_t(ld) * 2;
  if (!enabled || row_bytes > size_t(kXbMaxRowBytes) || (row_bytes & 15) || rows < 2 * sm_count() ||
      (reinterpret_cast<uintptr_t>(logits) & 15))
    return -100;
  const size_t smem = 2 * row_bytes + 128 + 256;
  static DeviceOnce configured;
  if (int e = configured.run([&] {
        return int(cudaFuncSetAttribute(xent_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        2 * kXbMaxRowBytes + 512));
      }))
    return e;
  XentBulkParams p;
  p.logits = static_cast<__nv_bfloat16*>(logits);
  p.targets = targets; p.losses = losses; p.lse_out = lse;
  p.rows = rows; p.vocab = vocab; p.ld = ld; p.scale = scale;
  p.ignore_index = ignore_index; p.write_grad = write_grad;
  p.st = status_device_ptr();
  const int grid = rows < sm_count() ? rows : sm_count();
  xent_bulk_kernel<<<grid, kXbThreads, smem, stream>>>(p);
  note_launches(1);
  return int(cudaGetLastError());
}

}  // namespace idrak
