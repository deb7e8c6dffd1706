// Token log-probability / entropy from logits, and its backward that rewrites the logits
// buffer into dlogits.  One CTA per row, single pass with an online softmax
// (running max m, Σe^{x−m}, Σx·e^{x−m}); the row is read exactly once in forward and once
// in backward.  Used per token-chunk behind the lm_head GEMM so that a full [T, V]
// logits tensor never exists.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace tk {

using bf16 = __nv_bfloat16;

struct Stat {
  float m, s, t;  // max, Σ e^{x−m}, Σ x e^{x−m}
};
__device__ __forceinline__ void stat_push(Stat& a, float x) {
  if (x > a.m) {
    const float c = __expf(a.m - x);
    a.s = a.s * c + 1.f;
    a.t = a.t * c + x;
    a.m = x;
  } else {
    const float e = __expf(x - a.m);
    a.s += e;
    a.t += x * e;
  }
}
__device__ __forceinline__ Stat stat_merge(const Stat& a, const Stat& b) {
  Stat r;
  r.m = fmaxf(a.m, b.m);
  const float ca = (a.m == -INFINITY) ? 0.f : __expf(a.m - r.m), cb = (b.m == -INFINITY) ? 0.f : __expf(b.m - r.m);
  r.s = a.s * ca + b.s * cb;
  r.t = a.t * ca + b.t * cb;
  return r;
}

// Eight values at once: their maximum first (no exponentials), one rescale of the running sums, then one exponential
// per value — 9/8 exponentials per element and no divergent branch (the per-element form above costs two per element
// once the lanes of a warp disagree on the branch, which bound the forward kernel on the special-function pipe).
__device__ __forceinline__ void stat_push8(Stat& a, const float (&x)[8]) {
  float vm = fmaxf(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])), fmaxf(fmaxf(x[4], x[5]), fmaxf(x[6], x[7])));
  const float m = fmaxf(a.m, vm);
  const float c = (a.m == -INFINITY) ? 0.f : __expf(a.m - m);
  float s = a.s * c, t = a.t * c;
  if (m != -INFINITY) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float e = __expf(x[i] - m);
      s += e;
      t += e > 0.f ? x[i] * e : 0.f;   // a masked (−inf) logit contributes nothing, not 0·inf
    }
  }
  a.m = m; a.s = s; a.t = t;
}

template <typename T>
__device__ __forceinline__ float ld1(const T* p) {
  if constexpr (std::is_same<T, float>::value) return *p; else return __bfloat162float(*p);
}

template <typename T>
__global__ void logprob_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ lp,
                                   float* __restrict__ lse, float* __restrict__ ent, int V, long ld, float inv_temp) {
  const long row = blockIdx.x;
  const T* x = logits + row * ld;
  Stat st{-INFINITY, 0.f, 0.f};
  constexpr int VEC = 16 / sizeof(T);
  const int nvec = (V / VEC);
  const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0);
  if (aligned) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 u = reinterpret_cast<const uint4*>(x)[v];
      if constexpr (std::is_same<T, float>::value) {
        stat_push(st, __uint_as_float(u.x) * inv_temp); stat_push(st, __uint_as_float(u.y) * inv_temp);
        stat_push(st, __uint_as_float(u.z) * inv_temp); stat_push(st, __uint_as_float(u.w) * inv_temp);
      } else {
        const uint32_t* pu = &u.x;
        float xv[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float2 a = unpack_bf16(pu[k]);
          xv[2 * k] = a.x * inv_temp;
          xv[2 * k + 1] = a.y * inv_temp;
        }
        stat_push8(st, xv);
      }
    }
    for (int i = nvec * VEC + threadIdx.x; i < V; i += blockDim.x) stat_push(st, ld1(x + i) * inv_temp);
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) stat_push(st, ld1(x + i) * inv_temp);
  }
  // block reduction
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Stat other{__shfl_xor_sync(0xffffffffu, st.m, o), __shfl_xor_sync(0xffffffffu, st.s, o), __shfl_xor_sync(0xffffffffu, st.t, o)};
    st = stat_merge(st, other);
  }
  __shared__ Stat sh[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sh[warp] = st;
  __syncthreads();
  if (warp == 0) {
    Stat a = lane < (blockDim.x >> 5) ? sh[lane] : Stat{-INFINITY, 0.f, 0.f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Stat other{__shfl_xor_sync(0xffffffffu, a.m, o), __shfl_xor_sync(0xffffffffu, a.s, o), __shfl_xor_sync(0xffffffffu, a.t, o)};
      a = stat_merge(a, other);
    }
    if (lane == 0) {
      const float l = a.m + __logf(a.s);
      const int64_t y = labels[row];
      const float xt = (y >= 0 && y < V) ? ld1(x + y) * inv_temp : 0.f;
      lp[row] = xt - l;
      lse[row] = l;
      if (ent) ent[row] = l - a.t / a.s;
    }
  }
}

// dlogits_j = [ glp·(δ_jy − p_j) − gent·p_j·(x_j − lse + H) ] / T   written over the logits buffer
template <typename T>
__global__ void logprob_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ labels, const float* __restrict__ lse,
                                   const float* __restrict__ ent, const float* __restrict__ glp, const float* __restrict__ gent, int V,
                                   long ld, float inv_temp) {
  const long row = blockIdx.x;
  T* x = logits + row * ld;
  const float l = lse[row], g = glp[row];
  const float ge = gent ? gent[row] : 0.f;
  const float mean_x = gent ? (l - ent[row]) : 0.f;  // E_p[x]
  const int64_t y = labels[row];
  constexpr int VEC = 16 / sizeof(T);
  const int nvec = V / VEC;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0);
  auto grad = [&](float raw, int j) -> float {
    const float xs = raw * inv_temp;
    const float p = __expf(xs - l);
    float d = g * ((j == y ? 1.f : 0.f) - p);
    if (gent) d -= ge * p * (xs - mean_x);
    return d * inv_temp;
  };
  if (aligned) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      uint4 u = reinterpret_cast<uint4*>(x)[v];
      const int j0 = v * VEC;
      if constexpr (std::is_same<T, float>::value) {
        u.x = __float_as_uint(grad(__uint_as_float(u.x), j0)); u.y = __float_as_uint(grad(__uint_as_float(u.y), j0 + 1));
        u.z = __float_as_uint(grad(__uint_as_float(u.z), j0 + 2)); u.w = __float_as_uint(grad(__uint_as_float(u.w), j0 + 3));
      } else {
        uint32_t* pu = &u.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float2 a = unpack_bf16(pu[k]);
          pu[k] = pack_bf16(grad(a.x, j0 + 2 * k), grad(a.y, j0 + 2 * k + 1));
        }
      }
      reinterpret_cast<uint4*>(x)[v] = u;
    }
    for (int i = nvec * VEC + threadIdx.x; i < V; i += blockDim.x) {
      float d = grad(ld1(x + i), i);
      if constexpr (std::is_same<T, float>::value) x[i] = d; else x[i] = __float2bfloat16(d);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float d = grad(ld1(x + i), i);
      if constexpr (std::is_same<T, float>::value) x[i] = d; else x[i] = __float2bfloat16(d);
    }
  }
}

std::vector<torch::Tensor> logprob_fwd(const torch::Tensor& logits, const torch::Tensor& labels, double temperature, bool with_entropy) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "logits [rows, V]");
  TORCH_CHECK(labels.scalar_type() == torch::kInt64 && labels.is_contiguous() && labels.numel() == logits.size(0), "labels int64 [rows]");
  c10::cuda::CUDAGuard guard(logits.device());
  const long rows = logits.size(0);
  const int V = logits.size(1);
  auto f32 = logits.options().dtype(torch::kFloat32);
  auto lp = torch::empty({rows}, f32), lse = torch::empty({rows}, f32);
  auto ent = with_entropy ? torch::empty({rows}, f32) : torch::empty({0}, f32);
  if (rows == 0) return {lp, lse, ent};
  auto stream = at::cuda::getCurrentCUDAStream();
  const float it = 1.f / static_cast<float>(temperature);
  if (logits.scalar_type() == torch::kBFloat16)
    logprob_fwd_kernel<bf16><<<rows, 256, 0, stream>>>(reinterpret_cast<const bf16*>(logits.data_ptr()), labels.data_ptr<int64_t>(),
                                                       lp.data_ptr<float>(), lse.data_ptr<float>(),
                                                       with_entropy ? ent.data_ptr<float>() : nullptr, V, logits.stride(0), it);
  else if (logits.scalar_type() == torch::kFloat32)
    logprob_fwd_kernel<float><<<rows, 256, 0, stream>>>(logits.data_ptr<float>(), labels.data_ptr<int64_t>(), lp.data_ptr<float>(),
                                                        lse.data_ptr<float>(), with_entropy ? ent.data_ptr<float>() : nullptr, V,
                                                        logits.stride(0), it);
  else TORCH_CHECK(false, "logits must be bf16 or fp32");
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {lp, lse, ent};
}

// Consumes `logits` (overwritten with dlogits) and returns it.
torch::Tensor logprob_bwd(torch::Tensor logits, const torch::Tensor& labels, const torch::Tensor& lse, const c10::optional<torch::Tensor>& ent,
                          const torch::Tensor& glp, const c10::optional<torch::Tensor>& gent, double temperature) {
  c10::cuda::CUDAGuard guard(logits.device());
  const long rows = logits.size(0);
  const int V = logits.size(1);
  if (rows == 0) return logits;
  const bool he = ent.has_value() && ent->defined() && gent.has_value() && gent->defined();
  auto stream = at::cuda::getCurrentCUDAStream();
  const float it = 1.f / static_cast<float>(temperature);
  if (logits.scalar_type() == torch::kBFloat16)
    logprob_bwd_kernel<bf16><<<rows, 256, 0, stream>>>(reinterpret_cast<bf16*>(logits.data_ptr()), labels.data_ptr<int64_t>(),
                                                       lse.data_ptr<float>(), he ? ent->data_ptr<float>() : nullptr, glp.data_ptr<float>(),
                                                       he ? gent->data_ptr<float>() : nullptr, V, logits.stride(0), it);
  else
    logprob_bwd_kernel<float><<<rows, 256, 0, stream>>>(logits.data_ptr<float>(), labels.data_ptr<int64_t>(), lse.data_ptr<float>(),
                                                        he ? ent->data_ptr<float>() : nullptr, glp.data_ptr<float>(),
                                                        he ? gent->data_ptr<float>() : nullptr, V, logits.stride(0), it);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return logits;
}

}  // namespace tk
