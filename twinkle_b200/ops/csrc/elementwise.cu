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
// One warp per row; lanes stride over 8-element vectors.  With `res` the row normalised is h = bf16(x + res), which is
// also written to `hsum` (the new residual stream): the add costs no pass of its own over the activations.
__global__ void rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, const bf16* __restrict__ w, bf16* __restrict__ y,
                                   bf16* __restrict__ hsum, float* __restrict__ rstd, int rows, int H, float eps, float offset) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    float ss = 0.f;
    if (res != nullptr) {
      const uint4* rr = reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * H);
      uint4* hr = reinterpret_cast<uint4*>(hsum + static_cast<size_t>(row) * H);
      for (int v = lane; v < nvec; v += 32) {
        const uint4 u = xr[v], q = rr[v];
        const uint32_t* pu = &u.x; const uint32_t* pq = &q.x;
        uint4 h;
        uint32_t* ph = &h.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 a = unpack_bf16(pu[k]), b = unpack_bf16(pq[k]);
          ph[k] = pack_bf16(a.x + b.x, a.y + b.y);
          const float2 c = unpack_bf16(ph[k]);  // the norm sees the rounded sum, as it would after a separate add
          ss += c.x * c.x + c.y * c.y;
        }
        hr[v] = h;
      }
      xr = hr;  // second pass: this lane re-reads the vectors it wrote itself
    } else {
      for (int v = lane; v < nvec; v += 32) {
        uint4 u = xr[v];
        float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
        ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
      }
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
// Row-block form (H ≤ 8192): the whole block works on the same R rows at a time and a thread owns the same VPT 16-byte
// column vectors in every row.  A row's g and x are read once into registers (2·R·VPT 16-byte loads per thread in
// flight), the row dot products are reduced warp → shared memory → warp with one block barrier per R rows (the
// partials are double-buffered), dx is produced from the registers, and dw lives in 8·VPT registers per thread for the
// whole kernel — one global atomic per column and block at the end.  `gadd` (optional) is a gradient that reaches the
// same tensor by another path (the residual stream): it is added to dx here instead of by a separate kernel.
template <int VPT, int R>
__global__ void __launch_bounds__(512, VPT == 1 ? 2 : 1)
    rmsnorm_bwd_rows_kernel(const bf16* __restrict__ g, const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ rstd,
                            const bf16* __restrict__ gadd, bf16* __restrict__ dx, float* __restrict__ dw, int rows, int H, float offset) {
  __shared__ float s_part[2][R][16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int nvec = H >> 3;
  const float inv_h = 1.f / H;
  float acc[VPT][8];
  uint4 wv[VPT];
  bool ok[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    ok[i] = v < nvec;
    wv[i] = ok[i] ? reinterpret_cast<const uint4*>(w)[v] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  }
  uint32_t wp[VPT][4];
#pragma unroll
  for (int i = 0; i < VPT; ++i) { wp[i][0] = wv[i].x; wp[i][1] = wv[i].y; wp[i][2] = wv[i].z; wp[i][3] = wv[i].w; }
  int buf = 0;
#pragma unroll 1
  for (long base = static_cast<long>(blockIdx.x) * R; base < rows; base += static_cast<long>(gridDim.x) * R, buf ^= 1) {
    uint32_t ux[R][VPT][4], ug[R][VPT][4];
    float r[R];
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const long row = base + q;
      const bool live = row < rows;
      r[q] = live ? rstd[row] : 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        uint4 tx = make_uint4(0u, 0u, 0u, 0u), tg = tx;
        if (live && ok[i]) {
          tx = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H)[v];
          tg = reinterpret_cast<const uint4*>(g + static_cast<size_t>(row) * H)[v];
        }
        ux[q][i][0] = tx.x; ux[q][i][1] = tx.y; ux[q][i][2] = tx.z; ux[q][i][3] = tx.w;
        ug[q][i][0] = tg.x; ug[q][i][1] = tg.y; ug[q][i][2] = tg.z; ug[q][i][3] = tg.w;
      }
    }
#pragma unroll
    for (int q = 0; q < R; ++q) {
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 a = unpack_bf16(ux[q][i][k]), b = unpack_bf16(ug[q][i][k]), c = unpack_bf16(wp[i][k]);
          dot += b.x * (c.x + offset) * a.x + b.y * (c.y + offset) * a.y;
        }
      }
      dot = warp_sum(dot);
      if (lane == 0) s_part[buf][q][warp] = dot;
    }
    __syncthreads();
    // the packed values stay the only copy kept across the barrier: without this fence the compiler holds the unpacked
    // fp32 values and products of the first pass for the second one, four times the registers
#pragma unroll
    for (int q = 0; q < R; ++q)
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) asm volatile("" : "+r"(ux[q][i][k]), "+r"(ug[q][i][k]));
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const long row = base + q;
      const float total = warp_sum(lane < nw ? s_part[buf][q][lane] : 0.f);
      const float rq = r[q], coef = total * rq * rq * inv_h;  // rq = 0 for rows past the end: nothing is added to dw
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const bool store = ok[i] && row < rows;
        uint4 ga = make_uint4(0u, 0u, 0u, 0u);  // bf16 zeros
        if (gadd != nullptr && store) ga = reinterpret_cast<const uint4*>(gadd + static_cast<size_t>(row) * H)[threadIdx.x + i * blockDim.x];
        const uint32_t pa[4] = {ga.x, ga.y, ga.z, ga.w};
        uint32_t po[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 a = unpack_bf16(ux[q][i][k]), b = unpack_bf16(ug[q][i][k]), c = unpack_bf16(wp[i][k]), e = unpack_bf16(pa[k]);
          po[k] = pack_bf16(rq * (b.x * (c.x + offset) - a.x * coef) + e.x, rq * (b.y * (c.y + offset) - a.y * coef) + e.y);
          acc[i][2 * k] += b.x * a.x * rq;
          acc[i][2 * k + 1] += b.y * a.y * rq;
        }
        if (store)
          reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * H)[threadIdx.x + i * blockDim.x] = make_uint4(po[0], po[1], po[2], po[3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (!ok[i]) continue;
    const int c0 = (threadIdx.x + i * blockDim.x) * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(&dw[c0 + e], acc[i][e]);
  }
}

// Wide rows (H > 8192): one warp per row.  Every warp keeps a private fp32 copy of dw in shared memory: lane l only ever
// touches the columns of its own 16-byte vectors, so the accumulation needs no atomics; the warps' copies are summed
// once at the end and added to the global result with one atomic per column and block.
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

// Returns {y, rstd} or, with a residual, {y, rstd, h} where h = x + residual is the row that was normalised.
std::vector<torch::Tensor> rmsnorm_fwd(const torch::Tensor& x, const torch::Tensor& w, double eps, double offset,
                                       const c10::optional<torch::Tensor>& residual) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.dim() == 2 && x.is_contiguous(), "x: [rows,H] bf16 contiguous");
  TORCH_CHECK(w.scalar_type() == torch::kBFloat16 && w.is_contiguous() && w.numel() == x.size(1), "w: [H] bf16");
  const int rows = x.size(0), H = x.size(1);
  TORCH_CHECK(H % 8 == 0, "H must be a multiple of 8");
  const bool has_res = residual.has_value() && residual->defined();
  if (has_res)
    TORCH_CHECK(residual->is_cuda() && residual->scalar_type() == torch::kBFloat16 && residual->is_contiguous() && residual->sizes() == x.sizes(),
                "residual: same shape as x, bf16 contiguous");
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty_like(x);
  auto rstd = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  torch::Tensor h = has_res ? torch::empty_like(x) : torch::Tensor();
  if (rows > 0) {
    int blocks = std::min((rows + 7) / 8, num_sms() * 8);
    rmsnorm_fwd_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const bf16*>(x.data_ptr()), has_res ? reinterpret_cast<const bf16*>(residual->data_ptr()) : nullptr,
        reinterpret_cast<const bf16*>(w.data_ptr()), reinterpret_cast<bf16*>(y.data_ptr()),
        has_res ? reinterpret_cast<bf16*>(h.data_ptr()) : nullptr, rstd.data_ptr<float>(), rows, H, static_cast<float>(eps),
        static_cast<float>(offset));
    count_launch();
    TK_CUDA_CHECK(cudaGetLastError());
  }
  if (has_res) return {y, rstd, h};
  return {y, rstd};
}

// `gadd` (optional, same shape as x): dx = gadd + the RMSNorm input gradient.
std::vector<torch::Tensor> rmsnorm_bwd(const torch::Tensor& g, const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& rstd,
                                       double offset, const c10::optional<torch::Tensor>& gadd) {
  const int rows = x.size(0), H = x.size(1);
  const bool has_add = gadd.has_value() && gadd->defined();
  if (has_add)
    TORCH_CHECK(gadd->is_cuda() && gadd->scalar_type() == torch::kBFloat16 && gadd->is_contiguous() && gadd->sizes() == x.sizes(),
                "gadd: same shape as x, bf16 contiguous");
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty_like(x);
  auto dw = torch::zeros({H}, x.options().dtype(torch::kFloat32));
  if (rows == 0) {
    if (has_add) dx.copy_(*gadd);
    return {dx, dw};
  }
  if (H <= 8192) {
    const int nvec = H / 8, vpt = nvec > 512 ? 2 : 1;
    const int threads = std::min(512, ((nvec + vpt - 1) / vpt + 31) / 32 * 32);
    constexpr int R = 2;
    const int blocks = static_cast<int>(std::max<long>(1, std::min<long>((rows + R - 1L) / R, num_sms() * (vpt == 1 ? 2L : 1L))));
    auto launch = [&](auto kern) {
      kern<<<blocks, threads, 0, at::cuda::getCurrentCUDAStream()>>>(
          reinterpret_cast<const bf16*>(g.data_ptr()), reinterpret_cast<const bf16*>(x.data_ptr()), reinterpret_cast<const bf16*>(w.data_ptr()),
          rstd.data_ptr<float>(), has_add ? reinterpret_cast<const bf16*>(gadd->data_ptr()) : nullptr, reinterpret_cast<bf16*>(dx.data_ptr()),
          dw.data_ptr<float>(), rows, H, static_cast<float>(offset));
    };
    if (vpt == 1) launch(rmsnorm_bwd_rows_kernel<1, R>); else launch(rmsnorm_bwd_rows_kernel<2, R>);
    count_launch();
    TK_CUDA_CHECK(cudaGetLastError());
    return {dx, dw};
  }
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
  if (has_add) dx.add_(*gadd);
  return {dx, dw};
}

// ------------------------------------------------------- q/k-norm + RoPE (D=128)
// One warp per token.  The token's fused row [heads, 128] is contiguous, so the warp walks it in 512-byte steps: each
// half-warp serves one head per step, lane j of the half holding elements [8j, 8j+8) with one 16-byte load; the
// rotate-half partner of element i (< 64) is i + 64, which lives in lane j ^ 8 of the same half.  cos / sin of the token
// are read once and kept in registers for all of its heads (read once per (token, head) they were two thirds of the
// kernel's memory traffic), no index needs a division, and ROPE_U loads per lane are issued before any arithmetic.
constexpr int ROPE_U = 4;

__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&x)[8]) {
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  return make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
}

template <bool HAS_NORM>
__global__ void __launch_bounds__(256, 3) qk_norm_rope_fwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                                                               const float* __restrict__ cosb, const float* __restrict__ sinb, bf16* __restrict__ q,
                                                               bf16* __restrict__ k, bf16* __restrict__ v, float* __restrict__ rstd, int T, int hq,
                                                               int hkv, float eps) {
  constexpr int D = 128;
  const int heads = hq + 2 * hkv;
  const int lane = threadIdx.x & 31, half = lane >> 4, j = lane & 15;
  const int fi = (j & 7) * 8;       // frequency index of this lane's first element
  const bool upper = j >= 8;        // elements 64..127
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  __shared__ float s_w[2][D];  // norm weights of q and k as fp32
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x)
    (&s_w[0][0])[i] = HAS_NORM ? __bfloat162float(i < D ? qw[i] : kw[i - D]) : 1.f;
  __syncthreads();
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < T; t += nwarps) {
    float cc[8], sn[8];
    {
      const float4 c0 = *reinterpret_cast<const float4*>(cosb + static_cast<size_t>(t) * 64 + fi);
      const float4 c1 = *reinterpret_cast<const float4*>(cosb + static_cast<size_t>(t) * 64 + fi + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sinb + static_cast<size_t>(t) * 64 + fi);
      const float4 s1 = *reinterpret_cast<const float4*>(sinb + static_cast<size_t>(t) * 64 + fi + 4);
      cc[0] = c0.x; cc[1] = c0.y; cc[2] = c0.z; cc[3] = c0.w; cc[4] = c1.x; cc[5] = c1.y; cc[6] = c1.z; cc[7] = c1.w;
      sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
      if (!upper) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sn[i] = -sn[i];  // o = x·cos − partner·sin below 64, + above
      }
    }
    const bf16* row = qkv + static_cast<size_t>(t) * heads * D + j * 8;
    for (int h0 = 0; h0 < heads; h0 += 2 * ROPE_U) {
      uint4 raw[ROPE_U];
#pragma unroll
      for (int u = 0; u < ROPE_U; ++u) {
        const int h = h0 + 2 * u + half;
        raw[u] = h < heads ? *reinterpret_cast<const uint4*>(row + static_cast<size_t>(h) * D) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < ROPE_U; ++u) {
        const int h = h0 + 2 * u + half;
        if (h0 + 2 * u >= heads) break;  // uniform over the warp
        // every lane runs the arithmetic (the shuffles need the whole warp); what is stored depends on the head's kind
        float xv[8];
        unpack8(raw[u], xv);
        const bool is_q = h < hq;
        if (HAS_NORM) {
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += xv[i] * xv[i];
          ss = half_warp_sum(ss);
          const float r = rsqrtf(ss / D + eps);
          const float* wsrc = &s_w[is_q ? 0 : 1][j * 8];
          const float4 w0 = *reinterpret_cast<const float4*>(wsrc), w1 = *reinterpret_cast<const float4*>(wsrc + 4);
          const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          if (j == 0 && h < hq + hkv) rstd[static_cast<size_t>(t) * (hq + hkv) + h] = r;
          // the reference path rounds the normalised value to bf16 before RoPE
#pragma unroll
          for (int i = 0; i < 8; ++i) xv[i] = __bfloat162float(__float2bfloat16(xv[i] * (r * wv[i])));
        }
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, xv[i], 8);
          o[i] = xv[i] * cc[i] + other * sn[i];
        }
        if (h >= heads) continue;
        if (h >= hq + hkv) {  // v: plain copy
          *reinterpret_cast<uint4*>(v + (static_cast<size_t>(t) * hkv + (h - hq - hkv)) * D + j * 8) = raw[u];
        } else {
          bf16* dst = is_q ? q + (static_cast<size_t>(t) * hq + h) * D : k + (static_cast<size_t>(t) * hkv + (h - hq)) * D;
          *reinterpret_cast<uint4*>(dst + j * 8) = pack8(o);
        }
      }
    }
  }
}

template <bool HAS_NORM>
__global__ void __launch_bounds__(256, 3) qk_norm_rope_bwd_kernel(const bf16* __restrict__ gq, const bf16* __restrict__ gk, const bf16* __restrict__ gv,
                                                               const bf16* __restrict__ qkv, const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                                                               const float* __restrict__ cosb, const float* __restrict__ sinb,
                                                               const float* __restrict__ rstd, bf16* __restrict__ dqkv, float* __restrict__ dqw,
                                                               float* __restrict__ dkw, int T, int hq, int hkv) {
  constexpr int D = 128;
  constexpr int U = 2;  // head pairs per round: 2·U 16-byte loads per lane are issued before the arithmetic
  __shared__ float s_dw[2][D];
  __shared__ float s_w[2][D];
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
    (&s_dw[0][0])[i] = 0.f;
    (&s_w[0][0])[i] = HAS_NORM ? __bfloat162float(i < D ? qw[i] : kw[i - D]) : 1.f;
  }
  __syncthreads();
  const int heads = hq + 2 * hkv;
  const int lane = threadIdx.x & 31, half = lane >> 4, j = lane & 15;
  const int fi = (j & 7) * 8;
  const bool upper = j >= 8;
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  float acc_w[2][8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc_w[0][i] = acc_w[1][i] = 0.f;
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < T; t += nwarps) {
    float cc[8], sn[8];
    {
      const float4 c0 = *reinterpret_cast<const float4*>(cosb + static_cast<size_t>(t) * 64 + fi);
      const float4 c1 = *reinterpret_cast<const float4*>(cosb + static_cast<size_t>(t) * 64 + fi + 4);
      const float4 s0 = *reinterpret_cast<const float4*>(sinb + static_cast<size_t>(t) * 64 + fi);
      const float4 s1 = *reinterpret_cast<const float4*>(sinb + static_cast<size_t>(t) * 64 + fi + 4);
      cc[0] = c0.x; cc[1] = c0.y; cc[2] = c0.z; cc[3] = c0.w; cc[4] = c1.x; cc[5] = c1.y; cc[6] = c1.z; cc[7] = c1.w;
      sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
      if (upper) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sn[i] = -sn[i];  // transpose of the forward rotation: + below 64, − above
      }
    }
    for (int h0 = 0; h0 < heads; h0 += 2 * U) {
      uint4 graw[U], raw[U];
      float rr[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = h0 + 2 * u + half;
        graw[u] = raw[u] = make_uint4(0u, 0u, 0u, 0u);
        rr[u] = 0.f;
        if (h < heads) {
          const bf16* gsrc = h < hq ? gq + (static_cast<size_t>(t) * hq + h) * D
                                    : (h < hq + hkv ? gk + (static_cast<size_t>(t) * hkv + (h - hq)) * D
                                                    : gv + (static_cast<size_t>(t) * hkv + (h - hq - hkv)) * D);
          graw[u] = *reinterpret_cast<const uint4*>(gsrc + j * 8);
          if (HAS_NORM && h < hq + hkv) {
            raw[u] = *reinterpret_cast<const uint4*>(qkv + (static_cast<size_t>(t) * heads + h) * D + j * 8);
            rr[u] = rstd[static_cast<size_t>(t) * (hq + hkv) + h];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int h = h0 + 2 * u + half;
        if (h0 + 2 * u >= heads) break;  // uniform over the warp
        const bool is_q = h < hq, is_v = h >= hq + hkv;
        float gy[8], gn[8];  // gn: gradient w.r.t. the (normalised) pre-RoPE value
        unpack8(graw[u], gy);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, gy[i], 8);
          gn[i] = gy[i] * cc[i] + other * sn[i];
        }
        uint4 outv;
        if (HAS_NORM) {
          float xv[8], wv[8];
          unpack8(raw[u], xv);
          const float* wsrc = &s_w[is_q ? 0 : 1][j * 8];
          const float4 w0 = *reinterpret_cast<const float4*>(wsrc), w1 = *reinterpret_cast<const float4*>(wsrc + 4);
          wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
          const float r = rr[u];
          float dot = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) dot += gn[i] * wv[i] * xv[i];
          dot = half_warp_sum(dot);
          const float coef = dot * r * r / D;
          float dx[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dx[i] = r * (gn[i] * wv[i] - xv[i] * coef);
            const float gw = gn[i] * xv[i] * r;  // zero for v heads and heads past the end (r = 0 there)
            acc_w[0][i] += is_q ? gw : 0.f;
            acc_w[1][i] += is_q ? 0.f : gw;
          }
          outv = pack8(dx);
        } else {
          outv = pack8(gn);
        }
        if (h >= heads) continue;
        *reinterpret_cast<uint4*>(dqkv + (static_cast<size_t>(t) * heads + h) * D + j * 8) = is_v ? graw[u] : outv;
      }
    }
  }
  if (HAS_NORM) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float a = acc_w[0][i] + __shfl_xor_sync(0xffffffffu, acc_w[0][i], 16);
      const float b = acc_w[1][i] + __shfl_xor_sync(0xffffffffu, acc_w[1][i], 16);
      if (half == 0) {
        atomicAdd(&s_dw[0][j * 8 + i], a);
        atomicAdd(&s_dw[1][j * 8 + i], b);
      }
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
  TORCH_CHECK(reinterpret_cast<uintptr_t>(qkv.data_ptr()) % 16 == 0, "qkv must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(qkv.device());
  const int T = qkv.size(0);
  auto q = torch::empty({T, hq, d}, qkv.options());
  auto k = torch::empty({T, hkv, d}, qkv.options());
  auto v = torch::empty({T, hkv, d}, qkv.options());
  auto rstd = torch::empty({T, hq + hkv}, qkv.options().dtype(torch::kFloat32));
  if (T == 0) return {q, k, v, rstd};
  int blocks = static_cast<int>(std::max<long>(1, std::min<long>((T + 7L) / 8, num_sms() * 8L)));
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
  int blocks = static_cast<int>(std::max<long>(1, std::min<long>((T + 7L) / 8, num_sms() * 8L)));
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
__device__ __forceinline__ void adamw_one(float& pi, float& mi, float& vi, float gi, float lr_wd, float b1, float b2, float eps,
                                          float step_size, float inv_sqrt_bc2, float omb1, float omb2) {
  // omb1 / omb2 = 1 − β formed in double on the host: 1.f − 0.999f is off by 5e-5 relative
  pi *= lr_wd;
  mi = b1 * mi + omb1 * gi;
  vi = b2 * vi + omb2 * (gi * gi);
  const float denom = sqrtf(vi) * inv_sqrt_bc2 + eps;
  pi -= step_size * __fdividef(mi, denom);
}

// Four elements per thread and iteration: 16-byte loads / stores of the fp32 state, 8- or 16-byte ones of the gradient and
// the working copy.  `vec` says that every pointer is 16-byte (bf16: 8-byte) aligned; the tail and unaligned calls take
// the scalar path.
template <typename GradT, typename OutT>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                                    const GradT* __restrict__ g, OutT* __restrict__ out, long n, float lr, float b1,
                                                    float b2, float eps, float wd, float bc1, float bc2, float gscale, int vec, float omb1,
                                                    float omb2) {
  const float lr_wd = 1.f - lr * wd, step_size = lr / bc1, inv_sqrt_bc2 = 1.f / sqrtf(bc2);
  const long tid = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x, nthreads = static_cast<long>(gridDim.x) * blockDim.x;
  const long n4 = vec ? (n >> 2) : 0;
  for (long q = tid; q < n4; q += nthreads) {
    float4 pp = reinterpret_cast<float4*>(p)[q], mm = reinterpret_cast<float4*>(m)[q], vv = reinterpret_cast<float4*>(v)[q];
    float gg[4];
    if constexpr (std::is_same<GradT, float>::value) {
      const float4 t = reinterpret_cast<const float4*>(g)[q];
      gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2*>(g)[q];
      const float2 a = unpack_bf16(t.x), b = unpack_bf16(t.y);
      gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
    }
    adamw_one<GradT, OutT>(pp.x, mm.x, vv.x, gg[0] * gscale, lr_wd, b1, b2, eps, step_size, inv_sqrt_bc2, omb1, omb2);
    adamw_one<GradT, OutT>(pp.y, mm.y, vv.y, gg[1] * gscale, lr_wd, b1, b2, eps, step_size, inv_sqrt_bc2, omb1, omb2);
    adamw_one<GradT, OutT>(pp.z, mm.z, vv.z, gg[2] * gscale, lr_wd, b1, b2, eps, step_size, inv_sqrt_bc2, omb1, omb2);
    adamw_one<GradT, OutT>(pp.w, mm.w, vv.w, gg[3] * gscale, lr_wd, b1, b2, eps, step_size, inv_sqrt_bc2, omb1, omb2);
    reinterpret_cast<float4*>(p)[q] = pp;
    reinterpret_cast<float4*>(m)[q] = mm;
    reinterpret_cast<float4*>(v)[q] = vv;
    if (out != nullptr) {
      if constexpr (std::is_same<OutT, float>::value) reinterpret_cast<float4*>(out)[q] = pp;
      else reinterpret_cast<uint2*>(out)[q] = make_uint2(pack_bf16(pp.x, pp.y), pack_bf16(pp.z, pp.w));
    }
  }
  for (long i = n4 * 4 + tid; i < n; i += nthreads) {
    float gi;
    if constexpr (std::is_same<GradT, float>::value) gi = g[i]; else gi = __bfloat162float(g[i]);
    float pi = p[i], mi = m[i], vi = v[i];
    adamw_one<GradT, OutT>(pi, mi, vi, gi * gscale, lr_wd, b1, b2, eps, step_size, inv_sqrt_bc2, omb1, omb2);
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
  const float bc1 = static_cast<float>(1.0 - std::pow(b1, static_cast<double>(step)));   // in double: 1 − β^t cancels badly in fp32
  const float bc2 = static_cast<float>(1.0 - std::pow(b2, static_cast<double>(step)));
  int blocks = static_cast<int>(std::min<long>((n / 4 + 255) / 256 + 1, num_sms() * 8L));
  auto stream = at::cuda::getCurrentCUDAStream();
  bf16* out_bf = nullptr;
  float* out_f = nullptr;
  if (out.has_value() && out->defined()) {
    TORCH_CHECK(out->numel() == n && out->is_contiguous(), "out size mismatch");
    if (out->scalar_type() == torch::kBFloat16) out_bf = reinterpret_cast<bf16*>(out->data_ptr());
    else if (out->scalar_type() == torch::kFloat32) { if (out->data_ptr() != master.data_ptr()) out_f = out->data_ptr<float>(); }
    else TORCH_CHECK(false, "out must be bf16 or fp32");
  }
  auto al = [](const void* q, size_t a) { return q == nullptr || reinterpret_cast<uintptr_t>(q) % a == 0; };
  const int vec = (al(master.data_ptr(), 16) && al(exp_avg.data_ptr(), 16) && al(exp_avg_sq.data_ptr(), 16) &&
                   al(grad.data_ptr(), grad.scalar_type() == torch::kFloat32 ? 16 : 8) && al(out_bf, 8) && al(out_f, 16)) ? 1 : 0;
#define TK_ADAM(GT, OT, OP)                                                                                                     \
  adamw_kernel<GT, OT><<<blocks, 256, 0, stream>>>(master.data_ptr<float>(), exp_avg.data_ptr<float>(), exp_avg_sq.data_ptr<float>(), \
      reinterpret_cast<const GT*>(grad.data_ptr()), OP, n, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, bc1, bc2, (float)gscale, vec, \
      (float)(1.0 - b1), (float)(1.0 - b2))
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
  const long tid = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x, nthreads = static_cast<long>(gridDim.x) * blockDim.x;
  constexpr int VEC = 16 / sizeof(T);
  const long nv = (reinterpret_cast<uintptr_t>(x) % 16 == 0) ? n / VEC : 0;    // 16-byte loads when the base allows it
  for (long q = tid; q < nv; q += nthreads) {
    const uint4 u = reinterpret_cast<const uint4*>(x)[q];
    if constexpr (std::is_same<T, float>::value) {
      const float a = __uint_as_float(u.x), b = __uint_as_float(u.y), c = __uint_as_float(u.z), d = __uint_as_float(u.w);
      acc += a * a + b * b + c * c + d * d;
    } else {
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
    }
  }
  for (long i = nv * VEC + tid; i < n; i += nthreads) {
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
