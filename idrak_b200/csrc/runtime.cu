// Process-wide runtime pieces shared by every kernel file: the host-mapped
// status word that bounded waits report into, the tensor-map encoder resolved
// from the driver at run time, and device attribute queries.
//
// Role in the reference: the CUDA driver binding and launcher checks
// (src/Idrak.Gpu/Cuda/CudaDriver.cs, CudaBackend.cs:2307-2396). Here the
// kernels are compiled ahead of time for sm_100a, so only the pieces a
// compiled library still needs at run time remain.
#include "common.cuh"
#include <cudaTypedefs.h>
#include <atomic>
#include <mutex>
#include <cstdio>
#include <cstring>

namespace idrak {

static Status* g_status_host = nullptr;
static Status* g_status_dev = nullptr;
static std::once_flag g_status_once;

static void init_status() {
  void* h = nullptr;
  if (cudaHostAlloc(&h, sizeof(Status), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  memset(h, 0, sizeof(Status));
  void* d = nullptr;
  if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
    cudaGetLastError();
    d = h;  // unified addressing: the host pointer is usable on the device
  }
  g_status_host = static_cast<Status*>(h);
  g_status_dev = static_cast<Status*>(d);
}

Status* status_device_ptr() {
  std::call_once(g_status_once, init_status);
  return g_status_dev;
}
Status* status_host_ptr() {
  std::call_once(g_status_once, init_status);
  return g_status_host;
}

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static void init_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess) {
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  } else {
    cudaGetLastError();
  }
}

static thread_local char g_last_error[512] = {0};
const char* last_error() { return g_last_error; }

int encode_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  std::call_once(g_encode_once, init_encode);
  if (!g_encode) return -1;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = g_encode(out, dtype, rank, base, gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_last_error, sizeof(g_last_error),
             "cuTensorMapEncodeTiled failed (%d): rank %d base %p dims [%llu,%llu,%llu,%llu] strides [%llu,%llu,%llu] "
             "box [%u,%u,%u,%u]",
             int(r), rank, base, (unsigned long long)gdim[0], (unsigned long long)(rank > 1 ? gdim[1] : 0),
             (unsigned long long)(rank > 2 ? gdim[2] : 0), (unsigned long long)(rank > 3 ? gdim[3] : 0),
             (unsigned long long)(rank > 1 ? gstr[0] : 0), (unsigned long long)(rank > 2 ? gstr[1] : 0),
             (unsigned long long)(rank > 3 ? gstr[2] : 0), bx[0], rank > 1 ? bx[1] : 0, rank > 2 ? bx[2] : 0,
             rank > 3 ? bx[3] : 0);
  }
  return r == CUDA_SUCCESS ? 0 : int(r);
}

static std::atomic<long long> g_launches{0};
void note_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

int sm_count() {
  static int cached[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

}  // namespace idrak

// Read and clear the status word. Returns the code (0 = no failure since the last call) and fills
// `out4` = {code, where, block, extra}.
IDRAK_API int idrak_status_take(uint32_t* out4) {
  idrak::Status* s = idrak::status_host_ptr();
  if (!s) return 0;
  uint32_t code = s->code;
  if (out4) {
    out4[0] = s->code;
    out4[1] = s->where;
    out4[2] = s->block;
    out4[3] = s->extra;
  }
  if (code) {
    s->where = 0;
    s->block = 0;
    s->extra = 0;
    __sync_synchronize();
    s->code = 0;
  }
  return int(code);
}

// Text describing the last failed host-side call on this thread (empty when none).
IDRAK_API const char* idrak_last_error() { return idrak::last_error(); }

IDRAK_API int idrak_sm_count() { return idrak::sm_count(); }

// Make `device`'s primary context current on the calling thread (threads PyTorch creates for the backward
// pass may not have one yet, and this library's driver-level calls need it).
IDRAK_API int idrak_bind_device(int device) { return int(cudaSetDevice(device)); }

// Kernels launched by this library in this process so far.
IDRAK_API long long idrak_launch_count() { return idrak::launches(); }

// The limits of the current device that the launchers size their grids, tiles and shared memory by, in this order:
//  0 SMs                         1 max threads per block          2 shared memory per block (opt-in), bytes
//  3 shared memory per SM        4 L2 bytes                       5 registers per SM
//  6 max resident blocks per SM  7 max resident threads per SM    8 warp size
//  9 memory bus width, bits     10 memory clock, kHz             11 SM clock, kHz
// 12 compute capability major   13 minor                         14 max cluster size the library uses (portable: 8)
// 15 tensor-memory columns per SM (512 on compute capability 10, else 0)
// Returns how many entries were written (at most `capacity`), or a negative CUDA error.
IDRAK_API int idrak_device_limits(long long* out, int capacity) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -int(e);
  const cudaDeviceAttr attrs[14] = {
      cudaDevAttrMultiProcessorCount, cudaDevAttrMaxThreadsPerBlock, cudaDevAttrMaxSharedMemoryPerBlockOptin,
      cudaDevAttrMaxSharedMemoryPerMultiprocessor, cudaDevAttrL2CacheSize, cudaDevAttrMaxRegistersPerMultiprocessor,
      cudaDevAttrMaxBlocksPerMultiprocessor, cudaDevAttrMaxThreadsPerMultiProcessor, cudaDevAttrWarpSize,
      cudaDevAttrGlobalMemoryBusWidth, cudaDevAttrMemoryClockRate, cudaDevAttrClockRate,
      cudaDevAttrComputeCapabilityMajor, cudaDevAttrComputeCapabilityMinor};
  long long v[16];
  for (int i = 0; i < 14; ++i) {
    int x = 0;
    e = cudaDeviceGetAttribute(&x, attrs[i], dev);
    if (e != cudaSuccess) return -int(e);
    v[i] = x;
  }
  v[14] = 8;
  v[15] = v[12] == 10 ? 512 : 0;
  const int n = capacity < 16 ? capacity : 16;
  for (int i = 0; i < n; ++i) out[i] = v[i];
  return n;
}

IDRAK_API const char* idrak_build_info() {
  return "idrak_b200 native kernels, sm_100a, built " __DATE__ " " __TIME__;
}
