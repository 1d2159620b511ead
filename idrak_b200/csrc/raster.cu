// Rasterisation and image-synthesis kernels that write into plain device buffers (no graphics API):
//   * exact area-coverage rasterisation of flattened outlines (glyphs, shapes): a signed-area accumulation pass over
//     line segments followed by a per-row prefix sum,
//   * the two passes of a separable resampling with precomputed tap tables - bit-exact with the 8-bit fixed-point
//     arithmetic Pillow uses (22 fractional bits, round half up, clip to 0..255), and a float variant,
//   * affine / perspective warps with nearest, bilinear and bicubic taps,
//   * box blur and rank (min / median / max) filters,
//   * one fused per-pixel pass for the scan / paper effects that need no neighbourhood (tone curve, vignette,
//     illumination gradient, counter-based Gaussian and salt-and-pepper noise, fibre texture).
// All are bandwidth-bound; one thread per output element (or per segment for the accumulation), grids sized from the
// element count and capped at a multiple of the SM count.
//
// Reference: the reference runs these on the CPU (src/Idrak.Imaging: CoverageRasterizer, PillowImageOps,
// PaperEffects.cs, PaperTransforms.cs); the coverage definition (signed trapezoid areas, non-zero or even-odd
// resolve) and the resampling arithmetic follow the same contracts.
#include "common.cuh"

namespace idrak {

static int raster_blocks(long long n, int per_sm = 16) {
  long long b = (n + 255) / 256, cap = (long long)sm_count() * per_sm;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

// ---------------------------------------------------------------------------------------------------------------
// Coverage accumulation. Each segment (x0, y0) -> (x1, y1) in pixel units, y down, belongs to image seg_image[i].
// For every pixel row the segment crosses, the piece inside the row is cut at the integer x positions; a piece
// inside cell c with signed height d and mean horizontal offset m (0..1 from the cell's left edge) adds
// d * (1 - m) to acc[c] and d * m to acc[c + 1]. After an inclusive prefix sum along the row, acc[c] is the signed
// area covered in cell c. Pieces left of the image fold into column 0 (they cover everything to their right);
// pieces right of it contribute nothing. acc has pitch >= W + 1 floats per row.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void add_piece(float* row, int W, float xa, float xb, float d) {
  // xa, xb inside one cell (or both outside the image on the same side)
  const float xm = 0.5f * (xa + xb);
  if (xm < 0.f) { atomicAdd(row, d); return; }
  if (xm >= float(W)) return;
  const int c = min(int(xm), W - 1);
  const float m = xm - float(c);
  atomicAdd(row + c, d * (1.f - m));
  atomicAdd(row + c + 1, d * m);
}

__global__ void __launch_bounds__(256) coverage_accumulate_kernel(const float4* __restrict__ segs,
                                                                  const int* __restrict__ seg_image, int n_segs,
                                                                  float* __restrict__ acc, int W, int H, int pitch) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_segs; i += gridDim.x * blockDim.x) {
    float4 s = segs[i];
    float x0 = s.x, y0 = s.y, x1 = s.z, y1 = s.w;
    if (y0 == y1) continue;
    float dir = 1.f;
    if (y0 > y1) { float t = x0; x0 = x1; x1 = t; t = y0; y0 = y1; y1 = t; dir = -1.f; }
    if (y1 <= 0.f || y0 >= float(H)) continue;
    const float dxdy = (x1 - x0) / (y1 - y0);
    float* img = acc + size_t(seg_image ? seg_image[i] : 0) * H * pitch;
    const int row_first = max(int(floorf(y0)), 0), row_last = min(int(ceilf(y1)) - 1, H - 1);
    for (int r = row_first; r <= row_last; ++r) {
      const float ya = fmaxf(y0, float(r)), yb = fminf(y1, float(r + 1));
      if (yb <= ya) continue;
      float xa = x0 + (ya - y0) * dxdy, xb = x0 + (yb - y0) * dxdy;
      const float d = (yb - ya) * dir;
      float* row = img + size_t(r) * pitch;
      if (xa > xb) { const float t = xa; xa = xb; xb = t; }
      // clip the piece to [0, W]: the parts outside keep their share of d
      const float span = xb - xa;
      if (span <= 0.f) { add_piece(row, W, xa, xb, d); continue; }
      const float inv = 1.f / span;
      if (xa < 0.f) {
        const float cut = fminf(xb, 0.f);
        atomicAdd(row, d * (cut - xa) * inv);
        xa = cut;
      }
      if (xb > float(W)) xb = fmaxf(xa, float(W));   // the part right of the image adds nothing
      // walk the cells between xa and xb
      float x = xa;
      while (x < xb) {
        const float next = fminf(floorf(x) + 1.f, xb);
        add_piece(row, W, x, next, d * (next - x) * inv);
        x = next;
      }
    }
  }
}

// One warp per row: inclusive scan of the row in 32-wide chunks with a carry, then |.| under the fill rule.
//   rule 0: non-zero winding (min(|a|, 1));  rule 1: even-odd (triangle wave of period 2)
template <typename T>
__global__ void __launch_bounds__(256) coverage_resolve_kernel(const float* __restrict__ acc, T* __restrict__ out,
                                                               long long rows, int W, int pitch, int rule) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += n_warps) {
    const float* a = acc + size_t(r) * pitch;
    T* o = out + size_t(r) * W;
    float carry = 0.f;
    for (int base = 0; base < W; base += 32) {
      const int c = base + lane;
      float v = c < W ? a[c] : 0.f;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v += u;
      }
      v += carry;
      carry = __shfl_sync(0xffffffffu, v, 31);
      float cov = fabsf(v);
      if (rule == 1) {
        cov = cov - 2.f * floorf(cov * 0.5f);
        if (cov > 1.f) cov = 2.f - cov;
      } else {
        cov = fminf(cov, 1.f);
      }
      if (c < W) {
        if constexpr (sizeof(T) == 1) o[c] = T(__float2int_rn(cov * 255.f));
        else o[c] = cov;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Separable resampling, one pass. The image is viewed as [outer, in_len, inner]; output [outer, out_len, inner]:
//   out[o, j, i] = sum_t in[o, lo[j] + t, i] * k[j * ksize + t],  t < count[j]
// 8-bit: k holds integers scaled by 2^22; the sum starts at 2^21 and is shifted down and clipped.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kPrecisionBits = 32 - 8 - 2;

__global__ void __launch_bounds__(256) resample_pass_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                                               const int* __restrict__ lo, const int* __restrict__ count,
                                                               const int* __restrict__ k, int ksize, long long outer,
                                                               int in_len, int out_len, long long inner) {
  const long long total = outer * out_len * inner;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long i = idx % inner;
    const int j = int((idx / inner) % out_len);
    const long long o = idx / (inner * out_len);
    const uint8_t* src = in + (o * in_len + lo[j]) * inner + i;
    const int* kk = k + size_t(j) * ksize;
    int ss = 1 << (kPrecisionBits - 1);
    const int n = count[j];
    for (int t = 0; t < n; ++t) ss += int(src[t * inner]) * kk[t];
    ss >>= kPrecisionBits;
    out[idx] = uint8_t(ss < 0 ? 0 : (ss > 255 ? 255 : ss));
  }
}

__global__ void __launch_bounds__(256) resample_pass_f32_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                const int* __restrict__ lo, const int* __restrict__ count,
                                                                const float* __restrict__ k, int ksize, long long outer,
                                                                int in_len, int out_len, long long inner) {
  const long long total = outer * out_len * inner;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long i = idx % inner;
    const int j = int((idx / inner) % out_len);
    const long long o = idx / (inner * out_len);
    const float* src = in + (o * in_len + lo[j]) * inner + i;
    const float* kk = k + size_t(j) * ksize;
    double ss = 0.0;
    const int n = count[j];
    for (int t = 0; t < n; ++t) ss += double(src[t * inner]) * double(kk[t]);
    out[idx] = float(ss);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Affine / perspective warp. For output pixel (x, y) the source position is
//   u = (a x' + b y' + c) / (g x' + h y' + 1),  v = (d x' + e y' + f) / (g x' + h y' + 1),  x' = x + 0.5, y' = y + 0.5
// (coefficients per image, 8 doubles). Taps: 0 nearest, 1 bilinear, 2 bicubic (the a = -1 cubic). Pixels whose source
// falls outside the image keep the fill value. Interleaved [B, H, W, C] in, [B, OH, OW, C] out. 8-bit results are
// truncated after the blend, as Pillow's transform does.
// ---------------------------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ T to_pixel(double v);
template <> __device__ __forceinline__ uint8_t to_pixel<uint8_t>(double v) {
  return v <= 0.0 ? uint8_t(0) : (v >= 255.0 ? uint8_t(255) : uint8_t(v));
}
template <> __device__ __forceinline__ float to_pixel<float>(double v) { return float(v); }

__device__ __forceinline__ int clipi(int v, int n) { return v < 0 ? 0 : (v >= n ? n - 1 : v); }

__device__ __forceinline__ double cubic_m1(double v1, double v2, double v3, double v4, double d) {
  const double p1 = v2, p2 = -v1 + v3, p3 = 2.0 * (v1 - v2) + v3 - v4, p4 = -v1 + v2 - v3 + v4;
  return p1 + d * (p2 + d * (p3 + d * p4));
}

template <typename T>
__global__ void __launch_bounds__(256) warp_kernel(const T* __restrict__ in, T* __restrict__ out,
                                                   const double* __restrict__ coef, const T* __restrict__ fill, int B, int H,
                                                   int W, int C, int OH, int OW, int taps) {
  const long long total = (long long)B * OH * OW;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int ox = int(idx % OW), oy = int((idx / OW) % OH), b = int(idx / ((long long)OW * OH));
    const double* m = coef + size_t(b) * 8;
    const double xs = ox + 0.5, ys = oy + 0.5;
    const double den = m[6] * xs + m[7] * ys + 1.0;
    double u = (m[0] * xs + m[1] * ys + m[2]) / den, v = (m[3] * xs + m[4] * ys + m[5]) / den;
    const T* img = in + size_t(b) * H * W * C;
    T* dst = out + size_t(idx) * C;
    const bool inside = u >= 0.0 && u < double(W) && v >= 0.0 && v < double(H);
    if (!inside) {
      for (int c = 0; c < C; ++c) dst[c] = fill ? fill[c] : T(0);
      continue;
    }
    if (taps == 0) {
      const int x = int(u), y = int(v);
      for (int c = 0; c < C; ++c) dst[c] = img[(size_t(y) * W + x) * C + c];
      continue;
    }
    u -= 0.5; v -= 0.5;
    const int x = int(floor(u)), y = int(floor(v));
    const double dx = u - x, dy = v - y;
    if (taps == 1) {
      const int x0 = clipi(x, W), x1 = clipi(x + 1, W), y0 = clipi(y, H);
      const bool has_y1 = (y + 1 >= 0 && y + 1 < H);
      for (int c = 0; c < C; ++c) {
        const double a = img[(size_t(y0) * W + x0) * C + c], bb = img[(size_t(y0) * W + x1) * C + c];
        const double r0 = a + (bb - a) * dx;
        double r1 = r0;
        if (has_y1) {
          const double d = img[(size_t(y + 1) * W + x0) * C + c], e = img[(size_t(y + 1) * W + x1) * C + c];
          r1 = d + (e - d) * dx;
        }
        dst[c] = to_pixel<T>(r0 + (r1 - r0) * dy);
      }
    } else {
      int xi[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) xi[t] = clipi(x - 1 + t, W);
      for (int c = 0; c < C; ++c) {
        double rows[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int yy = y - 1 + t;
          if (t != 1 && !(yy >= 0 && yy < H)) { rows[t] = 0.0; continue; }   // filled in below from a valid row
          const T* r = img + size_t(clipi(yy, H)) * W * C;
          rows[t] = cubic_m1(r[size_t(xi[0]) * C + c], r[size_t(xi[1]) * C + c], r[size_t(xi[2]) * C + c],
                             r[size_t(xi[3]) * C + c], dx);
        }
        // rows outside the image repeat their inner neighbour
        if (!(y - 1 >= 0 && y - 1 < H)) rows[0] = rows[1];
        if (!(y + 1 >= 0 && y + 1 < H)) rows[2] = rows[1];
        if (!(y + 2 >= 0 && y + 2 < H)) rows[3] = rows[2];
        dst[c] = to_pixel<T>(cubic_m1(rows[0], rows[1], rows[2], rows[3], dy));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Box blur (mean over a (2 rx + 1) x (2 ry + 1) window, edges replicated) and rank filter (the rank-th smallest of a
// k x k window, edges replicated) on interleaved 8-bit images. The rank is found by bisection on the value.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) box_blur_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int B,
                                                          int H, int W, int C, int rx, int ry) {
  const long long total = (long long)B * H * W * C;
  const int area = (2 * rx + 1) * (2 * ry + 1);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = int(idx % C), x = int((idx / C) % W), y = int((idx / ((long long)C * W)) % H);
    const int b = int(idx / ((long long)C * W * H));
    const uint8_t* img = in + size_t(b) * H * W * C;
    int sum = 0;
    for (int dy = -ry; dy <= ry; ++dy) {
      const uint8_t* row = img + size_t(clipi(y + dy, H)) * W * C;
      for (int dx = -rx; dx <= rx; ++dx) sum += row[size_t(clipi(x + dx, W)) * C + c];
    }
    out[idx] = uint8_t((2 * sum + area) / (2 * area));
  }
}

__global__ void __launch_bounds__(256) rank_filter_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int B,
                                                             int H, int W, int C, int k, int rank) {
  const long long total = (long long)B * H * W * C;
  const int r = k / 2;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = int(idx % C), x = int((idx / C) % W), y = int((idx / ((long long)C * W)) % H);
    const int b = int(idx / ((long long)C * W * H));
    const uint8_t* img = in + size_t(b) * H * W * C;
    int lo = 0, hi = 255;        // smallest value v with count(window <= v) > rank
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      int cnt = 0;
      for (int dy = -r; dy <= r; ++dy) {
        const uint8_t* row = img + size_t(clipi(y + dy, H)) * W * C;
        for (int dx = -r; dx <= r; ++dx) cnt += (row[size_t(clipi(x + dx, W)) * C + c] <= mid);
      }
      if (cnt > rank) hi = mid; else lo = mid + 1;
    }
    out[idx] = uint8_t(lo);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Fused per-pixel scan / paper effects on 8-bit interleaved images. Random numbers come from a counter-based
// hash of (seed, image, pixel, channel, stream), so results do not depend on the launch shape and a host
// restatement reproduces them.
// ---------------------------------------------------------------------------------------------------------------
struct EffectParams {
  float gain, bias, gamma;            // v = gain * v^gamma + bias, v in 0..1
  float grad_x, grad_y;               // illumination: v *= 1 + grad_x (x/W - 0.5) + grad_y (y/H - 0.5)
  float vignette, vignette_power;     // v *= 1 - vignette * r^power, r = distance from the centre / half diagonal
  float noise_sigma;                  // additive Gaussian, in 0..1 units
  float salt, pepper;                 // probabilities per pixel
  float fibre, fibre_scale;           // paper fibre: value noise of that amplitude, cells of 1 / scale pixels
  int same_noise_all_channels;        // 1: one draw per pixel (grey noise), 0: per channel
  unsigned long long seed;
};

__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long counter, unsigned stream) {
  const unsigned long long h = mix64(mix64(seed ^ (0xD1B54A32D192ED03ull * (stream + 1))) + counter);
  return float(h >> 40) * (1.0f / 16777216.0f);          // 24 bits -> [0, 1)
}
__device__ __forceinline__ float lattice(unsigned long long seed, int ix, int iy) {
  return uniform01(seed, (unsigned long long)(unsigned)ix * 0x1F123BB5ull + (unsigned long long)(unsigned)iy, 7u);
}

__global__ void __launch_bounds__(256) paper_effects_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int B,
                                                            int H, int W, int C, const EffectParams p) {
  const long long total = (long long)B * H * W * C;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = int(idx % C), x = int((idx / C) % W), y = int((idx / ((long long)C * W)) % H);
    const int b = int(idx / ((long long)C * W * H));
    float v = float(in[idx]) * (1.f / 255.f);
    if (p.gamma != 1.f) v = __powf(fmaxf(v, 0.f), p.gamma);
    v = p.gain * v + p.bias;
    const float fx = (x + 0.5f) / W - 0.5f, fy = (y + 0.5f) / H - 0.5f;
    v *= 1.f + p.grad_x * fx + p.grad_y * fy;
    if (p.vignette != 0.f) {
      const float r = sqrtf(fx * fx + fy * fy) * 1.41421356f;
      v *= 1.f - p.vignette * __powf(r, p.vignette_power);
    }
    if (p.fibre != 0.f) {
      const float gx = x * p.fibre_scale, gy = y * p.fibre_scale;
      const int ix = int(floorf(gx)), iy = int(floorf(gy));
      float tx = gx - ix, ty = gy - iy;
      tx = tx * tx * (3.f - 2.f * tx);
      ty = ty * ty * (3.f - 2.f * ty);
      const unsigned long long s = p.seed + b;
      const float n00 = lattice(s, ix, iy), n10 = lattice(s, ix + 1, iy), n01 = lattice(s, ix, iy + 1),
                  n11 = lattice(s, ix + 1, iy + 1);
      v += p.fibre * ((n00 + (n10 - n00) * tx) * (1.f - ty) + (n01 + (n11 - n01) * tx) * ty - 0.5f);
    }
    const unsigned long long pixel = ((unsigned long long)b * H + y) * W + x;
    const unsigned long long counter = p.same_noise_all_channels ? pixel : pixel * C + c;
    if (p.noise_sigma != 0.f) {
      const float u1 = fmaxf(uniform01(p.seed, counter, 1u), 5.9604645e-8f), u2 = uniform01(p.seed, counter, 2u);
      v += p.noise_sigma * sqrtf(-2.f * __logf(u1)) * __cosf(6.28318531f * u2);
    }
    if (p.salt != 0.f || p.pepper != 0.f) {
      const float u = uniform01(p.seed, pixel, 3u);
      if (u < p.pepper) v = 0.f;
      else if (u > 1.f - p.salt) v = 1.f;
    }
    out[idx] = uint8_t(__float2int_rn(fminf(fmaxf(v, 0.f), 1.f) * 255.f));
  }
}

}  // namespace idrak

using namespace idrak;

// ---------------------------------------------------------------------------------------------------------------
// C entry points (0 on success, a cudaError, or a negative argument error)
// ---------------------------------------------------------------------------------------------------------------
IDRAK_API int idrak_coverage_accumulate(const void* segs, const int* seg_image, int n_segs, float* acc, int W, int H,
                                        int pitch, void* stream_) {
  if (n_segs <= 0) return 0;
  if (W <= 0 || H <= 0 || pitch < W + 1) return -2;
  if (reinterpret_cast<uintptr_t>(segs) & 15) return -3;
  coverage_accumulate_kernel<<<raster_blocks(n_segs), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const float4*>(segs), seg_image, n_segs, acc, W, H, pitch);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_coverage_resolve(const float* acc, void* out, int out_u8, long long rows, int W, int pitch, int rule,
                                     void* stream_) {
  if (rows <= 0 || W <= 0) return 0;
  if (pitch < W) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int grid = raster_blocks(rows * 32);
  if (out_u8) coverage_resolve_kernel<uint8_t><<<grid, 256, 0, s>>>(acc, static_cast<uint8_t*>(out), rows, W, pitch, rule);
  else coverage_resolve_kernel<float><<<grid, 256, 0, s>>>(acc, static_cast<float*>(out), rows, W, pitch, rule);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_resample_pass(const void* in, void* out, int is_f32, const int* lo, const int* count, const void* k,
                                  int ksize, long long outer, int in_len, int out_len, long long inner, void* stream_) {
  if (outer <= 0 || out_len <= 0 || inner <= 0) return 0;
  if (in_len <= 0 || ksize <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int grid = raster_blocks(outer * out_len * inner);
  if (is_f32)
    resample_pass_f32_kernel<<<grid, 256, 0, s>>>(static_cast<const float*>(in), static_cast<float*>(out), lo, count,
                                                  static_cast<const float*>(k), ksize, outer, in_len, out_len, inner);
  else
    resample_pass_u8_kernel<<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), lo, count,
                                                 static_cast<const int*>(k), ksize, outer, in_len, out_len, inner);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_warp(const void* in, void* out, int is_f32, const double* coef, const void* fill, int B, int H, int W,
                         int C, int OH, int OW, int taps, void* stream_) {
  if (B <= 0 || OH <= 0 || OW <= 0) return 0;
  if (H <= 0 || W <= 0 || C <= 0 || taps < 0 || taps > 2) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int grid = raster_blocks((long long)B * OH * OW);
  if (is_f32)
    warp_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(in), static_cast<float*>(out), coef,
                                            static_cast<const float*>(fill), B, H, W, C, OH, OW, taps);
  else
    warp_kernel<uint8_t><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), coef,
                                              static_cast<const uint8_t*>(fill), B, H, W, C, OH, OW, taps);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_box_blur_u8(const void* in, void* out, int B, int H, int W, int C, int rx, int ry, void* stream_) {
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0) return 0;
  if (rx < 0 || ry < 0 || rx > 64 || ry > 64) return -2;
  box_blur_u8_kernel<<<raster_blocks((long long)B * H * W * C), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), B, H, W, C, rx, ry);
  note_launches(1);
  return int(cudaGetLastError());
}

IDRAK_API int idrak_rank_filter_u8(const void* in, void* out, int B, int H, int W, int C, int k, int rank, void* stream_) {
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0) return 0;
  if (k < 1 || k > 15 || (k & 1) == 0 || rank < 0 || rank >= k * k) return -2;
  rank_filter_u8_kernel<<<raster_blocks((long long)B * H * W * C), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), B, H, W, C, k, rank);
  note_launches(1);
  return int(cudaGetLastError());
}

// params: 13 floats in the order of EffectParams' float / int fields, then the seed separately
IDRAK_API int idrak_paper_effects(const void* in, void* out, int B, int H, int W, int C, const float* params,
                                  unsigned long long seed, void* stream_) {
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0) return 0;
  EffectParams p;
  p.gain = params[0]; p.bias = params[1]; p.gamma = params[2];
  p.grad_x = params[3]; p.grad_y = params[4];
  p.vignette = params[5]; p.vignette_power = params[6];
  p.noise_sigma = params[7];
  p.salt = params[8]; p.pepper = params[9];
  p.fibre = params[10]; p.fibre_scale = params[11];
  p.same_noise_all_channels = params[12] != 0.f;
  p.seed = seed;
  paper_effects_kernel<<<raster_blocks((long long)B * H * W * C), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), B, H, W, C, p);
  note_launches(1);
  return int(cudaGetLastError());
}
