// Column sums of a bf16 matrix without any allocation by the callee or the caller.
//
// This entry point has no counterpart in the reference: there every reduction takes its scratch from the
// device's buffer pool. It exists for callers that must not allocate at the moment of the call and have no
// workspace of their own to hand in - a host callback, a thread that must not take the allocator's lock, a
// C program that links this library without a tensor framework, a latency-critical loop where a device
// allocation would synchronise the whole device.
//
// The partial sums live in one array inside the library's device image, shared by every call on that device:
//   * capacity: idrak_colsum_static_max_floats() floats (1,048,576 = 4 MiB). A call needs
//     idrak_colsum_blocks(rows) * C of them (at most 128 * C), so every row count works for C <= 8192 and
//     wider matrices work when they have few rows. A call that needs more is refused with
//     IDRAK_COLSUM_STATIC_TOO_LARGE and a message (idrak_colsum_static_error()); nothing is launched.
//   * nothing in the array has to start at zero: each call writes every partial it later reads.
//   * two calls that overlap in time on one device (different streams, or different threads on streams that
//     are not ordered against each other) race on the array and produce garbage in both. Order them on one
//     stream or with events.
//   * the first call on each device looks the array's address up (with that device current) and keeps it.
//     Make that first call during start-up, outside any stream capture; later calls only launch kernels.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define IDRAK_COLSUM_STATIC_EXPORT __attribute__((visibility("default")))
#else
#define IDRAK_COLSUM_STATIC_EXPORT
#endif

#define IDRAK_COLSUM_STATIC_TOO_LARGE (-3)
#define IDRAK_COLSUM_STATIC_BAD_ARGUMENT (-2)

// out[c] (+)= sum over r of x[r, c], for x a bf16 matrix [rows, C] with `ld` elements between rows.
// `out` has C elements, fp32 when out_fp32 != 0 and bf16 otherwise; accumulate != 0 adds to what it holds.
// `stream` is a cudaStream_t (null = the default stream). The device that is current at the call is used.
// Returns 0, one of the codes above, or a positive cudaError_t.
IDRAK_COLSUM_STATIC_EXPORT int idrak_colsum_static(const void* x, int rows, int C, int ld, void* out, int out_fp32, int accumulate, void* stream);

// Capacity of the shared scratch array, in floats.
IDRAK_COLSUM_STATIC_EXPORT long long idrak_colsum_static_max_floats(void);

// Text of the last refusal or set-up failure of idrak_colsum_static on the calling thread ("" if none).
IDRAK_COLSUM_STATIC_EXPORT const char* idrak_colsum_static_error(void);

#ifdef __cplusplus
}
#endif
