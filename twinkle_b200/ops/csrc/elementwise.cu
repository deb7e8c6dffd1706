// Bandwidth-bound kernels: RMSNorm fwd/bwd, fused q/k-norm + RoPE fwd/bwd, SwiGLU fwd/bwd,
// fused AdamW, sum of squares.  All use 16-byte vector accesses; each tensor is read once
// (norm kernels re-read their row from L1 for the second pass) so DRAM traffic equals the
// algorithmic bytes.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace tk {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------ RMSNorm
// One warp per row; lanes stride over 8-element vectors.
__global__ void rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                                   float* __restrict__ rstd, int rows, int H, float eps, float offset) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      uint4 u = xr[v];
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / H + eps);
    if (lane == 0 && rstd) rstd[row] = r;
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    for (int v = lane; v < nvec; v += 32) {
      uint4 u = xr[v], ww = wr[v];
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      float2 wa = unpack_bf16(ww.x), wb = unpack_bf16(ww.y), wc = unpack_bf16(ww.z), wd = unpack_bf16(ww.w);
      uint4 o;
      o.x = pack_bf16(a.x * r * (wa.x + offset), a.y * r * (wa.y + offset));
      o.y = pack_bf16(b.x * r * (wb.x + offset), b.y * r * (wb.y + offset));
      o.z = pack_bf16(c.x * r * (wc.x + offset), c.y * r * (wc.y + offset));
      o.w = pack_bf16(d.x * r * (wd.x + offset), d.y * r * (wd.y + offset));
      yr[v] = o;
    }
  }
}

// dx = rstd·(g·w' − x·rstd²·mean(g·w'·x)),  dw += Σ_rows g·x·rstd.
// Every warp keeps a private fp32 copy of dw in shared memory: lane l only ever touches the columns of its own
// 16-byte vectors, so the accumulation needs no atomics; the warps' copies are summed once at the end and added to
// the global result with one atomic per column and block.
__global__ void rmsnorm_bwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                   const float* __restrict__ rstd, bf16* __restrict__ dx, float* __restrict__ dw, int rows, int H,
                                   float offset) {
  extern __shared__ float s_dw[];  // [warps][H]
  const int warps_per_block = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  float* my = s_dw + static_cast<size_t>(warp) * H;
  for (int v = lane; v < nvec; v += 32) {
    reinterpret_cast<float4*>(my)[2 * v] = make_float4(0.f, 0.f, 0.f, 0.f);
    reinterpret_cast<float4*>(my)[2 * v + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x * warps_per_block + warp; row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    const uint4* gr = reinterpret_cast<const uint4*>(g + static_cast<size_t>(row) * H);
    const float r = rstd[row];
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      uint4 ux = xr[v], ug = gr[v], uw = wr[v];
      const uint32_t* px = &ux.x; const uint32_t* pg = &ug.x; const uint32_t* pw = &uw.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 a = unpack_bf16(px[k]), b = unpack_bf16(pg[k]), c = unpack_bf16(pw[k]);
        dot += b.x * (c.x + offset) * a.x + b.y * (c.y + offset) * a.y;
      }
    }
    dot = warp_sum(dot);
    const float coef = dot * r * r / H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H);
    for (int v = lane; v < nvec; v += 32) {
      uint4 ux = xr[v], ug = gr[v], uw = wr[v], o;   // second read of the row comes from L1/L2
      const uint32_t* px = &ux.x; const uint32_t* pg = &ug.x; const uint32_t* pw = &uw.x; uint32_t* po = &o.x;
      float4 d0 = reinterpret_cast<float4*>(my)[2 * v], d1 = reinterpret_cast<float4*>(my)[2 * v + 1];
      float acc[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 a = unpack_bf16(px[k]), b = unpack_bf16(pg[k]), c = unpack_bf16(pw[k]);
        po[k] = pack_bf16(r * (b.x * (c.x + offset) - a.x * coef), r * (b.y * (c.y + offset) - a.y * coef));
        acc[2 * k] += b.x * a.x * r;
        acc[2 * k + 1] += b.y * a.y * r;
      }
      reinterpret_cast<float4*>(my)[2 * v] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      reinterpret_cast<float4*>(my)[2 * v + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      dxr[v] = o;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float t = 0.f;
    for (int wi = 0; wi < warps_per_block; ++wi) t += s_dw[static_cast<size_t>(wi) * H + i];
    atomicAdd(&dw[i], t);
  }
}

std::vector<torch::Tensor> rmsnorm_fwd(const torch::Tensor& x, const torch::Tensor& w, double eps, double offset) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.dim() == 2 && x.is_contiguous(), "x: [rows,H] bf16 contiguous");
  TORCH_CHECK(w.scalar_type() == torch::kBFloat16 && w.is_contiguous() && w.numel() == x.size(1), "w: [H] bf16");
  const int rows = x.size(0), H = x.size(1);
  TORCH_CHECK(H % 8 == 0, "H must be a multiple of 8");
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty_like(x);
  auto rstd = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  if (rows == 0) return {y, rstd};
  int blocks = std::min((rows + 7) / 8, num_sms() * 8);
  rmsnorm_fwd_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(x.data_ptr()), reinterpret_cast<const bf16*>(w.data_ptr()), reinterpret_cast<bf16*>(y.data_ptr()),
      rstd.data_ptr<float>(), rows, H, static_cast<float>(eps), static_cast<float>(offset));
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {y, rstd};
}

std::vector<torch::Tensor> rmsnorm_bwd(const torch::Tensor& g, const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& rstd,
                                       double offset) {
  const int rows = x.size(0), H = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty_like(x);
  auto dw = torch::zeros({H}, x.options().dtype(torch::kFloat32));
  if (rows == 0) return {dx, dw};
  // one private fp32 dw row per warp: as many warps as fit into shared memory (at most 8)
  int warps = 8;
  while (warps > 1 && static_cast<size_t>(warps) * H * sizeof(float) > 200 * 1024) warps >>= 1;
  const size_t smem = static_cast<size_t>(warps) * H * sizeof(float);
  TORCH_CHECK(smem <= 200 * 1024, "hidden size too large for the RMSNorm backward kernel");
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    TK_CUDA_CHECK(cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = 200 * 1024;
  }
  int blocks = std::min((rows + warps - 1) / warps, num_sms());
  rmsnorm_bwd_kernel<<<blocks, warps * 32, smem, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(g.data_ptr()), reinterpret_cast<const bf16*>(x.data_ptr()), reinterpret_cast<const bf16*>(w.data_ptr()),
      rstd.data_ptr<float>(), reinterpret_cast<bf16*>(dx.data_ptr()), dw.data_ptr<float>(), rows, H, static_cast<float>(offset));
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {dx, dw};
}

// ------------------------------------------------------- q/k-norm + RoPE (D=128)
// One warp per (token, head).  Lane l holds elements [4l, 4l+4); the rotate-half partner of
// element i (< 64) is i + 64, which lives in lane l ^ 16.
// Each warp takes ROPE_U consecutive (token, head) items per round and issues all their loads before any arithmetic:
// with one 256-byte load in flight per warp the kernel ran at a third of the memory bandwidth.
constexpr int ROPE_U = 4;

template <bool HAS_NORM>
__global__ void __launch_bounds__(256) qk_norm_rope_fwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                                                               const float* __restrict__ cosb, const float* __restrict__ sinb, bf16* __restrict__ q,
                                                               bf16* __restrict__ k, bf16* __restrict__ v, float* __restrict__ rstd, int T, int hq,
                                                               int hkv, float eps) {
  constexpr int D = 128;
  const int heads = hq + 2 * hkv;
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(T) * heads;
  const long nwarps = static_cast<long>(gridDim.x) * (blockDim.x >> 5);
  const int fi = (lane & 15) * 4;  // frequency index of this lane's first element
  float wq[4] = {1.f, 1.f, 1.f, 1.f}, wk[4] = {1.f, 1.f, 1.f, 1.f};
  if (HAS_NORM) {
    const uint2 a = *reinterpret_cast<const uint2*>(qw + lane * 4), b = *reinterpret_cast<const uint2*>(kw + lane * 4);
    const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y);
    wq[0] = a0.x; wq[1] = a0.y; wq[2] = a1.x; wq[3] = a1.y;
    wk[0] = b0.x; wk[1] = b0.y; wk[2] = b1.x; wk[3] = b1.y;
  }
  for (long base = (static_cast<long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * ROPE_U; base < total; base += nwarps * ROPE_U) {
    uint2 raw[ROPE_U];
    float4 cs[ROPE_U], sn4[ROPE_U];
    int tt[ROPE_U], hh[ROPE_U];
#pragma unroll
    for (int u = 0; u < ROPE_U; ++u) {
      const long item = base + u;
      tt[u] = -1;
      if (item < total) {
        tt[u] = static_cast<int>(item / heads);
        hh[u] = static_cast<int>(item - static_cast<long>(tt[u]) * heads);
        raw[u] = *reinterpret_cast<const uint2*>(qkv + static_cast<size_t>(item) * D + lane * 4);
        if (hh[u] < hq + hkv) {
          cs[u] = *reinterpret_cast<const float4*>(cosb + static_cast<size_t>(tt[u]) * 64 + fi);
          sn4[u] = *reinterpret_cast<const float4*>(sinb + static_cast<size_t>(tt[u]) * 64 + fi);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < ROPE_U; ++u) {
      if (tt[u] < 0) continue;  // uniform over the warp
      const int t = tt[u], h = hh[u];
      if (h >= hq + hkv) {  // v: plain copy
        *reinterpret_cast<uint2*>(v + (static_cast<size_t>(t) * hkv + (h - hq - hkv)) * D + lane * 4) = raw[u];
        continue;
      }
      float2 a = unpack_bf16(raw[u].x), b = unpack_bf16(raw[u].y);
      float xv[4] = {a.x, a.y, b.x, b.y};
      const bool is_q = h < hq;
      if (HAS_NORM) {
        float ss = warp_sum(xv[0] * xv[0] + xv[1] * xv[1] + xv[2] * xv[2] + xv[3] * xv[3]);
        const float r = rsqrtf(ss / D + eps);
        if (lane == 0) rstd[static_cast<size_t>(t) * (hq + hkv) + h] = r;
        // the reference path rounds the normalised value to bf16 before RoPE
#pragma unroll
        for (int i = 0; i < 4; ++i) xv[i] = __bfloat162float(__float2bfloat16(xv[i] * (r * (is_q ? wq[i] : wk[i]))));
      }
      const float cc[4] = {cs[u].x, cs[u].y, cs[u].z, cs[u].w}, sn[4] = {sn4[u].x, sn4[u].y, sn4[u].z, sn4[u].w};
      float o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, xv[i], 16);
        o[i] = (lane < 16) ? (xv[i] * cc[i] - other * sn[i]) : (xv[i] * cc[i] + other * sn[i]);
      }
      uint2 outv = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
      bf16* dst = is_q ? q + (static_cast<size_t>(t) * hq + h) * D : k + (static_cast<size_t>(t) * hkv + (h - hq)) * D;
      *reinterpret_cast<uint2*>(dst + lane * 4) = outv;
    }
  }
}

template <bool HAS_NORM>
__global__ void __launch_bounds__(256) qk_norm_rope_bwd_kernel(const bf16* __restrict__ gq, const bf16* __restrict__ gk, const bf16* __restrict__ gv,
                                                               const bf16* __restrict__ qkv, const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                                                               const float* __restrict__ cosb, const float* __restrict__ sinb,
                                                               const float* __restrict__ rstd, bf16* __restrict__ dqkv, float* __restrict__ dqw,
                                                               float* __restrict__ dkw, int T, int hq, int hkv) {
  constexpr int D = 128;
  constexpr int U = 2;  // items per warp per round, all loads issued before the arithmetic
  __shared__ float s_dw[2][D];
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&s_dw[0][0])[i] = 0.f;
  __syncthreads();
  const int heads = hq + 2 * hkv;
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(T) * heads;
  const long nwarps = static_cast<long>(gridDim.x) * (blockDim.x >> 5);
  const int fi = (lane & 15) * 4;
  float wq[4] = {1.f, 1.f, 1.f, 1.f}, wk[4] = {1.f, 1.f, 1.f, 1.f};
  if (HAS_NORM) {
    const uint2 a = *reinterpret_cast<const uint2*>(qw + lane * 4), b = *reinterpret_cast<const uint2*>(kw + lane * 4);
    const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y);
    wq[0] = a0.x; wq[1] = a0.y; wq[2] = a1.x; wq[3] = a1.y;
    wk[0] = b0.x; wk[1] = b0.y; wk[2] = b1.x; wk[3] = b1.y;
  }
  float acc_w[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  for (long base = (static_cast<long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * U; base < total; base += nwarps * U) {
    uint2 graw[U], raw[U];
    float4 cs[U], sn4[U];
    float rr[U];
    int tt[U], hh[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long item = base + u;
      tt[u] = -1;
      if (item < total) {
        const int t = static_cast<int>(item / heads), h = static_cast<int>(item - static_cast<long>(t) * heads);
        tt[u] = t; hh[u] = h;
        if (h >= hq + hkv) {
          graw[u] = *reinterpret_cast<const uint2*>(gv + (static_cast<size_t>(t) * hkv + (h - hq - hkv)) * D + lane * 4);
        } else {
          const bf16* gsrc = h < hq ? gq + (static_cast<size_t>(t) * hq + h) * D : gk + (static_cast<size_t>(t) * hkv + (h - hq)) * D;
          graw[u] = *reinterpret_cast<const uint2*>(gsrc + lane * 4);
          cs[u] = *reinterpret_cast<const float4*>(cosb + static_cast<size_t>(t) * 64 + fi);
          sn4[u] = *reinterpret_cast<const float4*>(sinb + static_cast<size_t>(t) * 64 + fi);
          if (HAS_NORM) {
            raw[u] = *reinterpret_cast<const uint2*>(qkv + static_cast<size_t>(item) * D + lane * 4);
            rr[u] = rstd[static_cast<size_t>(t) * (hq + hkv) + h];
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (tt[u] < 0) continue;  // uniform over the warp
      const int t = tt[u], h = hh[u];
      bf16* dst = dqkv + (static_cast<size_t>(t) * heads + h) * D + lane * 4;
      if (h >= hq + hkv) {
        *reinterpret_cast<uint2*>(dst) = graw[u];
        continue;
      }
      const bool is_q = h < hq;
      float2 ga = unpack_bf16(graw[u].x), gb = unpack_bf16(graw[u].y);
      const float gy[4] = {ga.x, ga.y, gb.x, gb.y};
      const float cc[4] = {cs[u].x, cs[u].y, cs[u].z, cs[u].w}, sn[4] = {sn4[u].x, sn4[u].y, sn4[u].z, sn4[u].w};
      float gn[4];  // gradient w.r.t. the (normalised) pre-RoPE value
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, gy[i], 16);
        gn[i] = (lane < 16) ? (gy[i] * cc[i] + other * sn[i]) : (gy[i] * cc[i] - other * sn[i]);
      }
      if (!HAS_NORM) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(gn[0], gn[1]), pack_bf16(gn[2], gn[3]));
        continue;
      }
      float2 xa = unpack_bf16(raw[u].x), xb = unpack_bf16(raw[u].y);
      const float xv[4] = {xa.x, xa.y, xb.x, xb.y};
      const float r = rr[u];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) dot += gn[i] * (is_q ? wq[i] : wk[i]) * xv[i];
      dot = warp_sum(dot);
      const float coef = dot * r * r / D;
      float dx[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dx[i] = r * (gn[i] * (is_q ? wq[i] : wk[i]) - xv[i] * coef);
        acc_w[is_q ? 0 : 1][i] += gn[i] * xv[i] * r;
      }
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(dx[0], dx[1]), pack_bf16(dx[2], dx[3]));
    }
  }
  if (HAS_NORM) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      atomicAdd(&s_dw[0][lane * 4 + i], acc_w[0][i]);
      atomicAdd(&s_dw[1][lane * 4 + i], acc_w[1][i]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      atomicAdd(&dqw[i], s_dw[0][i]);
      atomicAdd(&dkw[i], s_dw[1][i]);
    }
  }
}

std::vector<torch::Tensor> qk_norm_rope_fwd(const torch::Tensor& qkv, const torch::Tensor& qw, const torch::Tensor& kw,
                                            const torch::Tensor& cosb, const torch::Tensor& sinb, int64_t hq, int64_t hkv, int64_t d,
                                            double eps) {
  TORCH_CHECK(d == 128, "head_dim must be 128");
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == torch::kBFloat16 && qkv.is_contiguous() && qkv.dim() == 2, "qkv [T, heads*128] bf16");
  TORCH_CHECK(qkv.size(1) == (hq + 2 * hkv) * d, "qkv width mismatch");
  TORCH_CHECK(cosb.scalar_type() == torch::kFloat32 && cosb.is_contiguous() && cosb.size(1) == 64, "cos [T,64] fp32");
  c10::cuda::CUDAGuard guard(qkv.device());
  const int T = qkv.size(0);
  auto q = torch::empty({T, hq, d}, qkv.options());
  auto k = torch::empty({T, hkv, d}, qkv.options());
  auto v = torch::empty({T, hkv, d}, qkv.options());
  auto rstd = torch::empty({T, hq + hkv}, qkv.options().dtype(torch::kFloat32));
  if (T == 0) return {q, k, v, rstd};
  long items = static_cast<long>(T) * (hq + 2 * hkv);
  int blocks = static_cast<int>(std::max<long>(1, std::min<long>((items + 8 * ROPE_U - 1) / (8 * ROPE_U), num_sms() * 8L)));
  qk_norm_rope_fwd_kernel<true><<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(qkv.data_ptr()), reinterpret_cast<const bf16*>(qw.data_ptr()), reinterpret_cast<const bf16*>(kw.data_ptr()),
      cosb.data_ptr<float>(), sinb.data_ptr<float>(), reinterpret_cast<bf16*>(q.data_ptr()), reinterpret_cast<bf16*>(k.data_ptr()),
      reinterpret_cast<bf16*>(v.data_ptr()), rstd.data_ptr<float>(), T, hq, hkv, static_cast<float>(eps));
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {q, k, v, rstd};
}

std::vector<torch::Tensor> qk_norm_rope_bwd(const torch::Tensor& gq, const torch::Tensor& gk, const torch::Tensor& gv, const torch::Tensor& qkv,
                                            const torch::Tensor& qw, const torch::Tensor& kw, const torch::Tensor& cosb,
                                            const torch::Tensor& sinb, const torch::Tensor& rstd, int64_t hq, int64_t hkv, int64_t d) {
  c10::cuda::CUDAGuard guard(qkv.device());
  const int T = qkv.size(0);
  auto dqkv = torch::empty_like(qkv);
  auto dqw = torch::zeros({d}, qkv.options().dtype(torch::kFloat32));
  auto dkw = torch::zeros({d}, qkv.options().dtype(torch::kFloat32));
  if (T == 0) return {dqkv, dqw, dkw};
  long items = static_cast<long>(T) * (hq + 2 * hkv);
  int blocks = static_cast<int>(std::min<long>((items + 7) / 8, num_sms() * 8L));
  qk_norm_rope_bwd_kernel<true><<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(gq.data_ptr()), reinterpret_cast<const bf16*>(gk.data_ptr()), reinterpret_cast<const bf16*>(gv.data_ptr()),
      reinterpret_cast<const bf16*>(qkv.data_ptr()), reinterpret_cast<const bf16*>(qw.data_ptr()), reinterpret_cast<const bf16*>(kw.data_ptr()),
      cosb.data_ptr<float>(), sinb.data_ptr<float>(), rstd.data_ptr<float>(), reinterpret_cast<bf16*>(dqkv.data_ptr()),
      dqw.data_ptr<float>(), dkw.data_ptr<float>(), T, hq, hkv);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {dqkv, dqw, dkw};
}

// ----------------------------------------------------------- SwiGLU / GeGLU
// GELU = false: act(x) = x * sigmoid(x).  GELU = true: tanh-approximated GELU, act(x) = 0.5 x (1 + tanh(c (x + 0.044715 x^3))).
template <bool GELU>
__device__ __forceinline__ float glu_act(float x) {
  if (GELU) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return x / (1.f + __expf(-x));
}

// act(x) and d act / dx
template <bool GELU>
__device__ __forceinline__ float2 glu_act_grad(float x) {
  if (GELU) {
    const float x2 = x * x;
    const float t = tanhf(0.7978845608028654f * (x + 0.044715f * x * x2));
    const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x2);
    return make_float2(0.5f * x * (1.f + t), 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du);
  }
  const float s = 1.f / (1.f + __expf(-x));
  return make_float2(x * s, s * (1.f + x * (1.f - s)));
}

template <bool GELU>
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long rows, int I) {
  const int vec_per_row = I >> 3;
  const long total = rows * vec_per_row;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * I + c * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c * 8);
    const uint32_t* pg = &g.x; const uint32_t* pu = &u.x;
    uint4 o; uint32_t* po = &o.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = unpack_bf16(pg[k]), b = unpack_bf16(pu[k]);
      po[k] = pack_bf16(glu_act<GELU>(a.x) * b.x, glu_act<GELU>(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(out + r * I + c * 8) = o;
  }
}

template <bool GELU>
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ gy, const bf16* __restrict__ gu, bf16* __restrict__ dgu, long rows, int I) {
  const int vec_per_row = I >> 3;
  const long total = rows * vec_per_row;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row);
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * I + c * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c * 8);
    const uint4 y = *reinterpret_cast<const uint4*>(gy + r * I + c * 8);
    const uint32_t* pg = &g.x; const uint32_t* pu = &u.x; const uint32_t* py = &y.x;
    uint4 og, ou; uint32_t* pog = &og.x; uint32_t* pou = &ou.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = unpack_bf16(pg[k]), b = unpack_bf16(pu[k]), d = unpack_bf16(py[k]);
      const float2 f0 = glu_act_grad<GELU>(a.x), f1 = glu_act_grad<GELU>(a.y);
      pog[k] = pack_bf16(d.x * b.x * f0.y, d.y * b.y * f1.y);
      pou[k] = pack_bf16(d.x * f0.x, d.y * f1.x);
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + c * 8) = og;
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + I + c * 8) = ou;
  }
}

static torch::Tensor glu_fwd(const torch::Tensor& gu, bool gelu) {
  TORCH_CHECK(gu.is_cuda() && gu.scalar_type() == torch::kBFloat16 && gu.is_contiguous() && gu.dim() == 2, "gate_up [rows, 2I] bf16");
  const long rows = gu.size(0);
  const int I = gu.size(1) / 2;
  TORCH_CHECK(I % 8 == 0, "I must be a multiple of 8");
  c10::cuda::CUDAGuard guard(gu.device());
  auto out = torch::empty({rows, I}, gu.options());
  if (rows == 0) return out;
  long total = rows * (I / 8);
  int blocks = static_cast<int>(std::min<long>((total + 255) / 256, num_sms() * 16L));
  auto stream = at::cuda::getCurrentCUDAStream();
  const bf16* in = reinterpret_cast<const bf16*>(gu.data_ptr());
  bf16* o = reinterpret_cast<bf16*>(out.data_ptr());
  if (gelu) swiglu_fwd_kernel<true><<<blocks, 256, 0, stream>>>(in, o, rows, I);
  else swiglu_fwd_kernel<false><<<blocks, 256, 0, stream>>>(in, o, rows, I);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return out;
}

torch::Tensor swiglu_fwd(const torch::Tensor& gu) { return glu_fwd(gu, false); }
torch::Tensor geglu_fwd(const torch::Tensor& gu) { return glu_fwd(gu, true); }

static torch::Tensor glu_bwd(const torch::Tensor& gy, const torch::Tensor& gu, bool gelu) {
  TORCH_CHECK(gy.is_cuda() && gy.scalar_type() == torch::kBFloat16 && gy.is_contiguous() && gu.is_contiguous() && gy.dim() == 2 &&
              gy.size(0) == gu.size(0) && gy.size(1) * 2 == gu.size(1), "grad [rows, I] bf16 for gate_up [rows, 2I]");
  const long rows = gu.size(0);
  const int I = gu.size(1) / 2;
  c10::cuda::CUDAGuard guard(gu.device());
  auto dgu = torch::empty_like(gu);
  if (rows == 0) return dgu;
  long total = rows * (I / 8);
  int blocks = static_cast<int>(std::min<long>((total + 255) / 256, num_sms() * 16L));
  auto stream = at::cuda::getCurrentCUDAStream();
  const bf16* g = reinterpret_cast<const bf16*>(gy.data_ptr());
  const bf16* in = reinterpret_cast<const bf16*>(gu.data_ptr());
  bf16* o = reinterpret_cast<bf16*>(dgu.data_ptr());
  if (gelu) swiglu_bwd_kernel<true><<<blocks, 256, 0, stream>>>(g, in, o, rows, I);
  else swiglu_bwd_kernel<false><<<blocks, 256, 0, stream>>>(g, in, o, rows, I);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return dgu;
}

torch::Tensor swiglu_bwd(const torch::Tensor& gy, const torch::Tensor& gu) { return glu_bwd(gy, gu, false); }
torch::Tensor geglu_bwd(const torch::Tensor& gy, const torch::Tensor& gu) { return glu_bwd(gy, gu, true); }

// --------------------------------------------------------------------- AdamW
// fp32 master/moments; gradient fp32 or bf16, multiplied by grad_scale on read;
// optional bf16 (or fp32) working copy written in the same pass.
template <typename GradT, typename OutT>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const GradT* __restrict__ g,
                             OutT* __restrict__ out, long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                             float gscale) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float gi;
    if constexpr (std::is_same<GradT, float>::value) gi = g[i]; else gi = __bfloat162float(g[i]);
    gi *= gscale;
    float pi = p[i] * (1.f - lr * wd);
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    const float denom = sqrtf(vi / bc2) + eps;
    pi -= lr * (mi / bc1) / denom;
    p[i] = pi; m[i] = mi; v[i] = vi;
    if (out != nullptr) {
      if constexpr (std::is_same<OutT, float>::value) out[i] = pi; else out[i] = __float2bfloat16(pi);
    }
  }
}

void adamw_step(torch::Tensor master, torch::Tensor exp_avg, torch::Tensor exp_avg_sq, const torch::Tensor& grad,
                const c10::optional<torch::Tensor>& out, double lr, double b1, double b2, double eps, double wd, int64_t step,
                double gscale) {
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == torch::kFloat32 && master.is_contiguous(), "master fp32 contiguous");
  const long n = master.numel();
  TORCH_CHECK(grad.numel() == n && exp_avg.numel() == n && exp_avg_sq.numel() == n && grad.is_contiguous(), "size mismatch");
  if (n == 0) return;
  c10::cuda::CUDAGuard guard(master.device());
  const float bc1 = 1.f - static_cast<float>(std::pow(b1, static_cast<double>(step)));
  const float bc2 = 1.f - static_cast<float>(std::pow(b2, static_cast<double>(step)));
  int blocks = static_cast<int>(std::min<long>((n + 255) / 256, num_sms() * 16L));
  auto stream = at::cuda::getCurrentCUDAStream();
  bf16* out_bf = nullptr;
  float* out_f = nullptr;
  if (out.has_value() && out->defined()) {
    TORCH_CHECK(out->numel() == n && out->is_contiguous(), "out size mismatch");
    if (out->scalar_type() == torch::kBFloat16) out_bf = reinterpret_cast<bf16*>(out->data_ptr());
    else if (out->scalar_type() == torch::kFloat32) { if (out->data_ptr() != master.data_ptr()) out_f = out->data_ptr<float>(); }
    else TORCH_CHECK(false, "out must be bf16 or fp32");
  }
#define TK_ADAM(GT, OT, OP)                                                                                                     \
  adamw_kernel<GT, OT><<<blocks, 256, 0, stream>>>(master.data_ptr<float>(), exp_avg.data_ptr<float>(), exp_avg_sq.data_ptr<float>(), \
      reinterpret_cast<const GT*>(grad.data_ptr()), OP, n, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, bc1, bc2, (float)gscale)
  if (grad.scalar_type() == torch::kFloat32) {
    if (out_f) TK_ADAM(float, float, out_f); else TK_ADAM(float, bf16, out_bf);
  } else if (grad.scalar_type() == torch::kBFloat16) {
    if (out_f) TK_ADAM(bf16, float, out_f); else TK_ADAM(bf16, bf16, out_bf);
  } else {
    TORCH_CHECK(false, "grad must be fp32 or bf16");
  }
#undef TK_ADAM
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
}

// ------------------------------------------------------------------- Σ x²
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long n, float* __restrict__ out) {
  float acc = 0.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float v;
    if constexpr (std::is_same<T, float>::value) v = x[i]; else v = __bfloat162float(x[i]);
    acc += v * v;
  }
  acc = warp_sum(acc);
  __shared__ float s[32];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) atomicAdd(out, v);
  }
}

torch::Tensor sumsq(const torch::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be CUDA contiguous");
  c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::zeros({}, x.options().dtype(torch::kFloat32));
  const long n = x.numel();
  if (n == 0) return out;
  int blocks = static_cast<int>(std::min<long>((n + 1023) / 1024, num_sms() * 8L));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (x.scalar_type() == torch::kFloat32) sumsq_kernel<float><<<blocks, 256, 0, stream>>>(x.data_ptr<float>(), n, out.data_ptr<float>());
  else if (x.scalar_type() == torch::kBFloat16)
    sumsq_kernel<bf16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(x.data_ptr()), n, out.data_ptr<float>());
  else TORCH_CHECK(false, "sumsq: fp32 or bf16");
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return out;
}

}  // namespace tk
