// One launch between the packed QKV projection and attention: optional per-head RMS norm of queries and keys,
// rotary embedding of both, and the write of the new keys / values into the paged cache - bf16, or int8 with one
// scale per (token, kv head).
//
// The packed projection row of a token is [H query heads | Hkv key heads | Hkv value heads] x D. One warp takes one
// (token, head); lane l holds elements l, l + 32, l + 64, ... of the head, so both members of a rotation pair
// (i, i + rot_dim / 2) sit in the same lane.
//   query head   -> norm, rotate, written back in place (attention reads it from the projection buffer)
//   key head     -> norm, rotate, written back in place (prefill attention reads it there) and into the cache slot
//   value head   -> copied into the cache slot
// Replaces three launches of the unfused path (norm of q / k, RoPE, cache write).
//
// int8 cache: scale = max|x| / 127 per (token, kv head), code = round(x / scale); the decode attention kernel
// multiplies the scale back in (decode_attn.cu).
//
// Reference counterparts: norm_rope_heads_f32 (src/Idrak.Gpu/Cuda/PtxKernels.Decoder.cs:355-389), kv_write_bf16
// (PtxKernels.Decoding.cs:12), kv_write_int8 (PtxKernels.Quantized.cs:251).
#include "common.cuh"

namespace idrak {

struct NormRopeKvParams {
  __nv_bfloat16* qkv;            // [T, (H + 2 Hkv) D], rows row_stride elements apart
  long long row_stride;
  const int* positions;          // [T] or null (no rotation)
  const int* slots;              // [T]: block * block_size + offset, negative = do not cache; or null
  void* k_cache;                 // [slots, Hkv, D] bf16 or int8
  void* v_cache;
  float* k_scale;                // [slots, Hkv] when the cache is int8
  float* v_scale;
  const __nv_bfloat16* q_norm;   // [D] weights (already with any offset added) or null
  const __nv_bfloat16* k_norm;
  float eps;
  float theta, freq_scale;
  int rot_dim;                   // elements of a head that rotate (pairs i, i + rot_dim / 2); 0 = no rotation
  int T, H, Hkv, D, kv_int8;
};

// One warp per (token, head); each lane owns PER = D / 32 elements: index e = lane + 32 j.
template <int PER>
__global__ void __launch_bounds__(256) norm_rope_kv_kernel(const NormRopeKvParams p) {
  const int heads_total = p.H + 2 * p.Hkv;
  const long long unit = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)p.T * heads_total) return;
  const int t = int(unit / heads_total), h = int(unit - (long long)t * heads_total);
  const int lane = threadIdx.x & 31;
  const int D = p.D;
  __nv_bfloat16* src = p.qkv + size_t(t) * p.row_stride + size_t(h) * D;
  const bool is_q = h < p.H, is_k = !is_q && h < p.H + p.Hkv;
  const int kvh = is_q ? 0 : (is_k ? h - p.H : h - p.H - p.Hkv);
  float v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) v[j] = __bfloat162float(src[lane + 32 * j]);
  if (is_q || is_k) {
    const __nv_bfloat16* nw = is_q ? p.q_norm : p.k_norm;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) ss += v[j] * v[j];
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / float(D) + p.eps);
#pragma unroll
      for (int j = 0; j < PER; ++j)
        v[j] = __bfloat162float(__float2bfloat16(v[j] * r * __bfloat162float(nw[lane + 32 * j])));   // as a separate norm would store it
    }
    if (p.rot_dim > 0 && p.positions) {
      // element e < half pairs with e + half; with e = lane + 32 j the partner lives in the same lane at j + half / 32
      const int half = p.rot_dim >> 1;
      const int hj = half >> 5;                       // half % 32 == 0 (rot_dim % 64 == 0)
      const float pos = float(p.positions[t]) * p.freq_scale;      // the arithmetic of rope_kernel, so results agree bit for bit
#pragma unroll
      for (int j = 0; j < PER / 2; ++j) {
        if (j < hj) {
          const int e = lane + 32 * j;
          const float inv = __powf(p.theta, -2.0f * float(e) / float(p.rot_dim));
          float sn, cs;
          sincosf(pos * inv, &sn, &cs);
          const float a = v[j], b = v[j + hj];
          v[j] = a * cs - b * sn;
          v[j + hj] = b * cs + a * sn;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) src[lane + 32 * j] = __float2bfloat16(v[j]);
  }
  if (is_q || !p.slots) return;
  const int slot = p.slots[t];
  if (slot < 0) return;
  const size_t row = (size_t(slot) * p.Hkv + kvh) * D;
  if (!p.kv_int8) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(is_k ? p.k_cache : p.v_cache) + row;
#pragma unroll
    for (int j = 0; j < PER; ++j) dst[lane + 32 * j] = __float2bfloat16(v[j]);
  } else {
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      v[j] = __bfloat162float(__float2bfloat16(v[j]));       // quantise what the bf16 cache would have held
      mx = fmaxf(mx, fabsf(v[j]));
    }
    mx = warp_max(mx);
    const float scale = mx > 0.f ? mx / 127.f : 1.f;
    int8_t* dst = static_cast<int8_t*>(is_k ? p.k_cache : p.v_cache) + row;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int q = __float2int_rn(v[j] / scale);
      dst[lane + 32 * j] = int8_t(max(-127, min(127, q)));
    }
    if (lane == 0) (is_k ? p.k_scale : p.v_scale)[size_t(slot) * p.Hkv + kvh] = scale;
  }
}

}  // namespace idrak

using namespace idrak;

// qkv rows are rotated / normalised in place; keys and values also go to the cache rows named by `slots`.
// Needs D in {64, 128, 256} and rot_dim % 64 == 0 (0: no rotation). Returns 0, a CUDA error or a negative
// argument error.
IDRAK_API int idrak_norm_rope_kv(void* qkv, long long row_stride, const int* positions, const int* slots, void* k_cache,
                                 void* v_cache, float* k_scale, float* v_scale, const void* q_norm, const void* k_norm,
                                 float eps, float theta, float freq_scale, int rot_dim, int T, int H, int Hkv, int D,
                                 int kv_int8, void* stream_) {
  if (T <= 0) return 0;
  if (D != 64 && D != 128 && D != 256) return -2;
  if (rot_dim < 0 || rot_dim > D || (rot_dim & 63)) return -3;
  if (kv_int8 && slots && (!k_scale || !v_scale)) return -4;
  NormRopeKvParams p;
  p.qkv = static_cast<__nv_bfloat16*>(qkv);
  p.row_stride = row_stride;
  p.positions = positions; p.slots = slots;
  p.k_cache = k_cache; p.v_cache = v_cache; p.k_scale = k_scale; p.v_scale = v_scale;
  p.q_norm = static_cast<const __nv_bfloat16*>(q_norm);
  p.k_norm = static_cast<const __nv_bfloat16*>(k_norm);
  p.eps = eps; p.theta = theta; p.freq_scale = freq_scale; p.rot_dim = rot_dim;
  p.T = T; p.H = H; p.Hkv = Hkv; p.D = D; p.kv_int8 = kv_int8;
  const long long units = (long long)T * (H + 2 * Hkv);
  const int blocks = int((units + 7) / 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  if (D == 64) norm_rope_kv_kernel<2><<<blocks, 256, 0, s>>>(p);
  else if (D == 128) norm_rope_kv_kernel<4><<<blocks, 256, 0, s>>>(p);
  else norm_rope_kv_kernel<8><<<blocks, 256, 0, s>>>(p);
  note_launches(1);
  return int(cudaGetLastError());
}
