// Column sums with the partial sums in a fixed array of the library's own device image: the call allocates
// nothing and the caller supplies no workspace. See colsum_static.h for who needs that and for the rules of
// sharing one array between calls.
//
// The arithmetic is that of idrak_colsum (rowops.cu), step for step: the rows are cut into the same number of
// chunks, inside a chunk eight row lanes stride the rows and are folded in lane order, and the chunk sums are
// folded in the same fixed order - so both entry points give the same bits for the same input.
#include "colsum_static.h"

#include <cstdio>
#include <mutex>

#include "common.cuh"

extern "C" int idrak_colsum_blocks(int rows);     // rowops.cu: how many row chunks idrak_colsum uses

namespace idrak {
namespace {

constexpr long long kStaticScratchFloats = 1ll << 20;     // 4 MiB
constexpr int kMaxDevices = 64;

// Shared by every idrak_colsum_static call on this device. Nothing here needs an initial value.
static __device__ __align__(256) float g_colsum_static_scratch[kStaticScratchFloats];

float* g_scratch_of_device[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;
thread_local char g_error[384] = {0};

// One block = 32 column lanes x 8 row lanes over a chunk of rows; a column lane owns 8 neighbouring columns.
// `vector_ok` (16-byte aligned rows) picks one 128-bit load per row over eight scalar loads.
__global__ void __launch_bounds__(256) colsum_static_part_kernel(const __nv_bfloat16* __restrict__ x, int rows, int C,
                                                                 int ld, int rows_per_block, int vector_ok,
                                                                 float* __restrict__ part) {
  __shared__ float sm[8][256];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + tx * 8;
  const int row0 = blockIdx.y * rows_per_block;
  const int row1 = min(rows, row0 + rows_per_block);
  float a[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = 0.f;
  if (vector_ok && col + 8 <= C) {
    for (int r = row0 + ty; r < row1; r += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + size_t(r) * ld + col);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        a[2 * j] += f.x;
        a[2 * j + 1] += f.y;
      }
    }
  } else if (col < C) {
    const int n = min(8, C - col);
    for (int r = row0 + ty; r < row1; r += 8)
      for (int j = 0; j < n; ++j) a[j] += __bfloat162float(x[size_t(r) * ld + col + j]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[ty][tx * 8 + j] = a[j];
  __syncthreads();
  const int c = threadIdx.x;
  if (blockIdx.x * 256 + c < C) {
    float r = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) r += sm[k][c];
    part[size_t(blockIdx.y) * C + blockIdx.x * 256 + c] = r;
  }
}

// out[c] (+)= sum_p part[p, c]: lane ty adds chunks ty, ty + 8, ... in ascending order, then the eight lane
// sums are added in lane order.
__global__ void __launch_bounds__(256) colsum_static_final_kernel(const float* __restrict__ part, int parts, int C,
                                                                  void* __restrict__ out, int out_fp32,
                                                                  int accumulate) {
  __shared__ float sm[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < C)
    for (int p = ty; p < parts; p += 8) s += part[size_t(p) * C + c];
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < C) {
    float r = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) r += sm[k][tx];
    if (out_fp32) {
      float* o = static_cast<float*>(out);
      o[c] = accumulate ? o[c] + r : r;
    } else {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
      o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + r : r);
    }
  }
}

// The scratch array's address on the current device; looked up once per device, with that device current.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    snprintf(g_error, sizeof(g_error), "idrak_colsum_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    return int(e);
  }
  if (dev < 0 || dev >= kMaxDevices) {
    snprintf(g_error, sizeof(g_error), "idrak_colsum_static: device %d is outside the supported range 0..%d", dev,
             kMaxDevices - 1);
    return IDRAK_COLSUM_STATIC_BAD_ARGUMENT;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_of_device[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_colsum_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      snprintf(g_error, sizeof(g_error), "idrak_colsum_static: cudaGetSymbolAddress failed on device %d: %s", dev,
               cudaGetErrorString(e));
      return e != cudaSuccess ? int(e) : IDRAK_COLSUM_STATIC_BAD_ARGUMENT;
    }
    g_scratch_of_device[dev] = ptr;
  }
  *out = g_scratch_of_device[dev];
  return 0;
}

}  // namespace
}  // namespace idrak

using namespace idrak;

IDRAK_API long long idrak_colsum_static_max_floats(void) { return kStaticScratchFloats; }

IDRAK_API const char* idrak_colsum_static_error(void) { return g_error; }

IDRAK_API int idrak_colsum_static(const void* x, int rows, int C, int ld, void* out, int out_fp32, int accumulate,
                                  void* stream_) {
  g_error[0] = 0;
  if (x == nullptr || out == nullptr || rows <= 0 || C <= 0 || ld < C) {
    snprintf(g_error, sizeof(g_error),
             "idrak_colsum_static: bad argument (x=%p out=%p rows=%d C=%d ld=%d; need rows > 0, C > 0, ld >= C)", x, out,
             rows, C, ld);
    return IDRAK_COLSUM_STATIC_BAD_ARGUMENT;
  }
  const int parts = idrak_colsum_blocks(rows);
  const long long need = static_cast<long long>(parts) * C;
  if (need > kStaticScratchFloats) {
    snprintf(g_error, sizeof(g_error),
             "idrak_colsum_static: %d rows x %d columns need %lld scratch floats (%d row chunks x %d); the built-in "
             "array holds %lld. Use idrak_colsum with a workspace of your own for this size.",
             rows, C, need, parts, C, kStaticScratchFloats);
    return IDRAK_COLSUM_STATIC_TOO_LARGE;
  }
  float* part = nullptr;
  const int rc = scratch_for_current_device(&part);
  if (rc != 0) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int rows_per_block = (rows + parts - 1) / parts;
  const int vector_ok = (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  dim3 grid((C + 255) / 256, parts);
  colsum_static_part_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), rows, C, ld, rows_per_block,
                                                vector_ok, part);
  colsum_static_final_kernel<<<(C + 31) / 32, 256, 0, s>>>(part, parts, C, out, out_fp32, accumulate);
  note_launches(2);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    snprintf(g_error, sizeof(g_error), "idrak_colsum_static: launch failed: %s", cudaGetErrorString(e));
  return int(e);
}
