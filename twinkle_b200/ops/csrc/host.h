// Host-side utilities shared by the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#define TK_CUDA_CHECK(expr)                                                                              \
  do {                                                                                                   \
    cudaError_t _e = (expr);                                                                             \
    TORCH_CHECK(_e == cudaSuccess, "CUDA error ", cudaGetErrorString(_e), " at ", __FILE__, ":", __LINE__); \
  } while (0)

namespace tk {

// Launch counter: every kernel launch issued by this extension bumps it (read by benchmarks).
void count_launch(int n = 1);
long launch_count();

// Number of SMs of the current device (cached).
int num_sms();

// Device int (per device) that kernels set when a bounded wait expires.  0 = healthy.
int* error_word();
// Reads (synchronising) and clears the error word; returns its value.
int read_and_clear_error();

// 2-D bf16 tensor map over a row-major matrix: `inner` contiguous elements per row, `outer` rows,
// `row_stride` elements between rows; the box is box_inner × box_outer with 128-byte swizzle.
CUtensorMap make_tmap_2d(const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride, uint32_t box_inner,
                         uint32_t box_outer, int elem_bytes = 2, bool swizzle128 = true);
// 3-D variant: dims {d0 (contiguous), d1, d2} with strides (in elements) s1, s2.
CUtensorMap make_tmap_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t b0,
                         uint32_t b1, uint32_t b2, int elem_bytes = 2, bool swizzle128 = true);

}  // namespace tk
