// C ABI entry point that allocates nothing.  It has no counterpart in the reference project (which ships no
// native code); it exists for callers that cannot ask an allocator for scratch at call time:
//   * hosts outside PyTorch that reach this library through dlopen / ctypes and have no caching allocator, and
//   * training loops whose device memory is planned to the last buffer, where a cudaMalloc inside the backward
//     pass would synchronise the device and may fail.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest hidden size the static scratch serves (fp32 words; 32 KiB of device memory per device).
#define TK_NOALLOC_MAX_H 8192

// RMSNorm backward: dx = rstd·(g·(w+offset) − x·rstd²·mean(g·(w+offset)·x)) (bf16) and dw = Σ_rows g·x·rstd (fp32).
//   g, x [rows, H] bf16 row-major; w [H] bf16; rstd [rows] fp32; dx [rows, H] bf16; dw [H] fp32 (overwritten).
//   H must be a multiple of 8 and ≤ TK_NOALLOC_MAX_H; all pointers 16-byte aligned device memory of the current device.
// The weight-gradient accumulator and a completion ticket live in file-scope __device__ storage that starts at zero
// (module load) and that every call returns to zero before it ends, so nothing is allocated, zeroed or freed by the host.
// The first call on a device does the set-up (symbol address look-up, SM count); make that call before any stream
// capture begins.  Calls on one device share the scratch: two calls that overlap in time (different streams or
// threads) race — issue them on one stream or order them with events.
// Two host threads that both make the first call on a device at the same moment both run the set-up; they write the
// same values, so the outcome is the same, but the set-up is not otherwise synchronised — if the first call may come
// from several threads, make one call up front.  The scratch is guaranteed to be back at zero only after a call
// that returned 0 has completed on the device: after −3 (launch failed) or a kernel that was aborted, its contents
// are unspecified and the next result may be wrong until the library is reloaded.
// Returns 0, or a negative code: −1 bad shape / alignment, −2 set-up failed, −3 launch failed (see tk_noalloc_strerror).
int tk_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd, void* dx, float* dw, int rows, int H,
                           float offset, cudaStream_t stream);

const char* tk_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
