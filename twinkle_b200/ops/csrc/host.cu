// Host utilities: SM count, per-device error word, TMA descriptor encoding through the
// driver entry point (no link-time dependency on libcuda).
#include <c10/cuda/CUDAGuard.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "host.h"

namespace tk {

static std::atomic<long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long launch_count() { return g_launches.load(std::memory_order_relaxed); }

int num_sms() {
  static std::vector<int> cache(64, 0);
  int dev = 0;
  TK_CUDA_CHECK(cudaGetDevice(&dev));
  if (cache[dev] == 0) {
    cudaDeviceProp prop;
    TK_CUDA_CHECK(cudaGetDeviceProperties(&prop, dev));
    cache[dev] = prop.multiProcessorCount;
  }
  return cache[dev];
}

static std::mutex g_mu;
static std::vector<int*> g_err(64, nullptr);

int* error_word() {
  int dev = 0;
  TK_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_err[dev] == nullptr) {
    TK_CUDA_CHECK(cudaMalloc(&g_err[dev], 64));
    TK_CUDA_CHECK(cudaMemset(g_err[dev], 0, 64));
  }
  return g_err[dev];
}

int read_and_clear_error() {
  int* p = error_word();
  int v = 0;
  TK_CUDA_CHECK(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) TK_CUDA_CHECK(cudaMemset(p, 0, sizeof(int)));
  return v;
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    TK_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    TORCH_CHECK(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled not available in this driver");
    fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

static CUtensorMapDataType dtype_of(int elem_bytes) {
  return elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
}

CUtensorMap make_tmap_2d(const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride, uint32_t box_inner,
                         uint32_t box_outer, int elem_bytes, bool swizzle128) {
  CUtensorMap m;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0 && strides[0] % 16 == 0, "TMA: base and row pitch must be 16-byte aligned");
  CUresult r = encode_fn()(&m, dtype_of(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(2d) failed with code ", static_cast<int>(r), " dims=", inner, "x", outer,
              " pitch=", strides[0], " box=", box_inner, "x", box_outer);
  return m;
}

CUtensorMap make_tmap_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t b0,
                         uint32_t b1, uint32_t b2, int elem_bytes, bool swizzle128) {
  CUtensorMap m;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * static_cast<uint64_t>(elem_bytes), s2 * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0 && strides[0] % 16 == 0 && strides[1] % 16 == 0,
              "TMA: base and pitches must be 16-byte aligned");
  CUresult r = encode_fn()(&m, dtype_of(elem_bytes), 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled(3d) failed with code ", static_cast<int>(r));
  return m;
}

}  // namespace tk
