// Allocation-free variant of the RMSNorm backward kernel behind a plain C entry point (see noalloc.h).
// Only the CUDA runtime is used: no torch, no cudaMalloc / cudaFree, no library routine that allocates.
#include "noalloc.h"

#include <cuda_bf16.h>
#include <stdint.h>

namespace {

constexpr int kMaxDevices = 64;

// Scratch: fp32 weight-gradient accumulator + completion ticket.  Zero at module load; each launch's last
// block writes the result out and puts both back to zero.
static __device__ __align__(256) float g_dw_scratch[TK_NOALLOC_MAX_H];
static __device__ __align__(256) unsigned int g_ticket[64];

struct DeviceState {
  bool ready = false;
  float* scratch = nullptr;
  unsigned int* ticket = nullptr;
  int sms = 0;
};
DeviceState g_state[kMaxDevices];

__device__ __forceinline__ float2 unpack2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256) rmsnorm_bwd_noalloc_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, float* scratch,
                                                                   unsigned int* ticket, int rows, int H, float offset) {
  extern __shared__ float s_dw[];
  __shared__ bool s_last;
  for (int i = threadIdx.x; i < H; i += blockDim.x) s_dw[i] = 0.f;
  __syncthreads();
  const int warps_per_block = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    const uint4* gr = reinterpret_cast<const uint4*>(g + static_cast<size_t>(row) * H);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    const float r = rstd[row];
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      uint4 ux = xr[v], ug = gr[v], uw = wr[v];
      const uint32_t* px = &ux.x; const uint32_t* pg = &ug.x; const uint32_t* pw = &uw.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 a = unpack2(px[k]), b = unpack2(pg[k]), c = unpack2(pw[k]);
        dot += b.x * (c.x + offset) * a.x + b.y * (c.y + offset) * a.y;
      }
    }
    dot = warp_sum_f(dot);
    const float coef = dot * r * r / H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H);
    for (int v = lane; v < nvec; v += 32) {
      uint4 ux = xr[v], ug = gr[v], uw = wr[v], o;
      const uint32_t* px = &ux.x; const uint32_t* pg = &ug.x; const uint32_t* pw = &uw.x; uint32_t* po = &o.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 a = unpack2(px[k]), b = unpack2(pg[k]), c = unpack2(pw[k]);
        po[k] = pack2(r * (b.x * (c.x + offset) - a.x * coef), r * (b.y * (c.y + offset) - a.y * coef));
        atomicAdd(&s_dw[v * 8 + 2 * k], b.x * a.x * r);
        atomicAdd(&s_dw[v * 8 + 2 * k + 1], b.y * a.y * r);
      }
      dxr[v] = o;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) atomicAdd(&scratch[i], s_dw[i]);
  // last block to finish publishes the sums and restores the scratch to zero
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    __threadfence();
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      dw[i] = __ldcg(&scratch[i]);
      scratch[i] = 0.f;
    }
    if (threadIdx.x == 0) *ticket = 0u;
  }
}

int setup_device(int dev) {
  DeviceState& st = g_state[dev];
  if (st.ready) return 0;
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_dw_scratch) != cudaSuccess || p == nullptr) return -2;
  st.scratch = static_cast<float*>(p);
  if (cudaGetSymbolAddress(&p, g_ticket) != cudaSuccess || p == nullptr) return -2;
  st.ticket = static_cast<unsigned int*>(p);
  if (cudaDeviceGetAttribute(&st.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || st.sms <= 0) return -2;
  st.ready = true;
  return 0;
}

}  // namespace

extern "C" int tk_rmsnorm_bwd_noalloc(const void* g, const void* x, const void* w, const float* rstd, void* dx, float* dw, int rows, int H,
                                      float offset, cudaStream_t stream) {
  if (rows < 0 || H <= 0 || H % 8 != 0 || H > TK_NOALLOC_MAX_H) return -1;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
                         reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dw) | reinterpret_cast<uintptr_t>(rstd);
  if (!g || !x || !w || !rstd || !dx || !dw || (bits & 15u)) return -1;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -2;
  if (int rc = setup_device(dev)) return rc;
  const DeviceState& st = g_state[dev];
  int blocks = (rows + 7) / 8;
  if (blocks > st.sms * 2) blocks = st.sms * 2;
  if (blocks < 1) blocks = 1;  // rows == 0: one block still writes dw = 0
  rmsnorm_bwd_noalloc_kernel<<<blocks, 256, H * sizeof(float), stream>>>(
      static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), rstd,
      static_cast<__nv_bfloat16*>(dx), dw, st.scratch, st.ticket, rows, H, offset);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" const char* tk_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "bad argument: H must be a multiple of 8 and at most TK_NOALLOC_MAX_H (8192); pointers non-null and 16-byte aligned";
    case -2: return "set-up failed: cudaGetSymbolAddress / device query returned an error";
    case -3: return "kernel launch failed";
    default: return "unknown code";
  }
}
