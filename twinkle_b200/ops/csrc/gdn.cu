// Gated DeltaNet (linear attention) kernels: depth-wise causal conv1d (+SiLU) over packed sequences and the gated
// delta-rule recurrence with the q/k L2 normalisation and the grouped-head repeat folded in.
//
//   S_t = α_t · S_{t-1} + k̂_t δ_tᵀ ,  δ_t = β_t (v_t − α_t S_{t-1}ᵀ k̂_t) ,  o_t = S_tᵀ q̂_t        (S ∈ R^{dk×dv}, fp32)
//
// What the reference gets from FLA's Triton kernels (src/twinkle/model/transformers/strategy/sequence_parallel/
// linear_attention_sp.py:266-308: causal_conv1d → chunk_gated_delta_rule).
//
// Recurrence layout: one WARP per (sequence, value head, 32 value columns).  Lane j owns column j of the state — all dk
// rows of it, in registers — so S ᵀk̂ and S ᵀq̂ are thread-local dot products and the rank-1 update is one FMA per
// element: no cross-thread reduction inside the time loop.  The state columns of a head are independent of one another,
// which is what lets a head be split over dv/32 warps.  k̂, q̂ of the next GDN_CH tokens are normalised co-operatively
// (one warp reduction per token) and staged in shared memory as fp32; the inner loop reads them as broadcast float4.
// Rewriting o_t = α·(S_{t-1}ᵀq̂) + δ·(q̂·k̂) lets both dot products run in the single pass over the old state.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace tk {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------ causal conv1d (+ SiLU), packed sequences
// x [T, C] (row stride xs), w [C, W], y [T, C] contiguous.  One thread per (token, 8 channels).  seg_start[t] = first
// token of t's sequence (the window never reaches across it).
template <int W>
__global__ void __launch_bounds__(256) causal_conv1d_fwd_kernel(const bf16* __restrict__ x, long xs, const bf16* __restrict__ w,
                                                                const int* __restrict__ seg_start, bf16* __restrict__ y, int T, int C,
                                                                int act) {
  const int cv = C >> 3;
  const long total = static_cast<long>(T) * cv;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / cv), c0 = static_cast<int>(idx - static_cast<long>(t) * cv) * 8;
    const int s0 = seg_start[t];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const int tt = t - (W - 1 - j);
      if (tt < s0) continue;
      const uint4 u = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(tt) * xs + c0);
      const uint32_t pu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = unpack_bf16(pu[e]);
        acc[2 * e] += a.x * __bfloat162float(w[static_cast<size_t>(c0 + 2 * e) * W + j]);
        acc[2 * e + 1] += a.y * __bfloat162float(w[static_cast<size_t>(c0 + 2 * e + 1) * W + j]);
      }
    }
    if (act) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = acc[e] / (1.f + __expf(-acc[e]));
    }
    *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * C + c0) =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

torch::Tensor causal_conv1d_fwd(const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& seg_start, bool activation) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "x: [T, C] bf16, unit channel stride");
  TORCH_CHECK(w.scalar_type() == torch::kBFloat16 && w.is_contiguous() && w.dim() == 2 && w.size(0) == x.size(1), "w: [C, W] bf16");
  TORCH_CHECK(seg_start.scalar_type() == torch::kInt32 && seg_start.is_contiguous() && seg_start.numel() == x.size(0), "seg_start: [T] int32");
  const int T = x.size(0), C = x.size(1), W = w.size(1);
  TORCH_CHECK(C % 8 == 0 && x.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "channels in 16-byte vectors");
  TORCH_CHECK(W >= 2 && W <= 4, "kernel width 2..4");
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({T, C}, x.options());
  if (T == 0) return y;
  const long total = static_cast<long>(T) * (C / 8);
  const int blocks = static_cast<int>(std::min<long>((total + 255) / 256, num_sms() * 8L));
  auto stream = at::cuda::getCurrentCUDAStream();
  auto launch = [&](auto kern) {
    kern<<<blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(x.data_ptr()), x.stride(0), reinterpret_cast<const bf16*>(w.data_ptr()),
                                     seg_start.data_ptr<int>(), reinterpret_cast<bf16*>(y.data_ptr()), T, C, activation ? 1 : 0);
  };
  if (W == 4) launch(causal_conv1d_fwd_kernel<4>);
  else if (W == 3) launch(causal_conv1d_fwd_kernel<3>);
  else launch(causal_conv1d_fwd_kernel<2>);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return y;
}

// ------------------------------------------------------------------ gated delta rule, recurrent form
constexpr int GDN_CH = 8;  // tokens normalised and staged per round

template <int DK>
__global__ void __launch_bounds__(32) gdn_recurrent_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                               long qs, long ks, long vs,  // token strides (elements)
                                                               const float* __restrict__ g, const float* __restrict__ beta,  // [T, Hv]
                                                               const int* __restrict__ cu, const float* __restrict__ init_state,
                                                               bf16* __restrict__ o, float* __restrict__ final_state, int Hv, int rep,
                                                               int dv, float scale) {
  __shared__ __align__(16) float s_k[GDN_CH][DK];
  __shared__ __align__(16) float s_q[GDN_CH][DK];
  __shared__ float s_qk[GDN_CH];
  const int lane = threadIdx.x;
  const int seq = blockIdx.z, h = blockIdx.y, col = blockIdx.x * 32 + lane;
  const int hk = h / rep;
  const int t0 = cu[seq], t1 = cu[seq + 1];
  float S[DK];
  const size_t st_off = ((static_cast<size_t>(seq) * Hv + h) * DK) * dv + col;
  if (init_state != nullptr && col < dv) {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = init_state[st_off + static_cast<size_t>(i) * dv];
  } else {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = 0.f;
  }
  constexpr int EPL = DK / 32;  // elements of a q / k row per lane while staging
  for (int tb = t0; tb < t1; tb += GDN_CH) {
    const int n = min(GDN_CH, t1 - tb);
    __syncwarp();
    float kv_[GDN_CH][EPL], qv_[GDN_CH][EPL];
#pragma unroll
    for (int c = 0; c < GDN_CH; ++c) {  // all loads of the round first
      const bf16* kr = k + static_cast<size_t>(tb + c) * ks + static_cast<size_t>(hk) * DK + lane * EPL;
      const bf16* qr = q + static_cast<size_t>(tb + c) * qs + static_cast<size_t>(hk) * DK + lane * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        kv_[c][e] = c < n ? __bfloat162float(kr[e]) : 0.f;
        qv_[c][e] = c < n ? __bfloat162float(qr[e]) : 0.f;
      }
    }
#pragma unroll
    for (int c = 0; c < GDN_CH; ++c) {
      float sk = 0.f, sq = 0.f, dqk = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        sk += kv_[c][e] * kv_[c][e];
        sq += qv_[c][e] * qv_[c][e];
        dqk += kv_[c][e] * qv_[c][e];
      }
      sk = warp_sum(sk); sq = warp_sum(sq); dqk = warp_sum(dqk);
      const float rk = rsqrtf(sk + 1e-6f), rq = scale * rsqrtf(sq + 1e-6f);   // x / sqrt(Σx² + 1e-6), the FLA convention
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        s_k[c][lane * EPL + e] = kv_[c][e] * rk;
        s_q[c][lane * EPL + e] = qv_[c][e] * rq;
      }
      if (lane == 0) s_qk[c] = dqk * rk * rq;
    }
    // lane c carries token c's scalars; they are handed to the whole warp by shuffle inside the loop
    float my_a = 1.f, my_b = 0.f;
    if (lane < n) {
      my_a = __expf(g[static_cast<size_t>(tb + lane) * Hv + h]);
      my_b = beta[static_cast<size_t>(tb + lane) * Hv + h];
    }
    __syncwarp();
    for (int c = 0; c < n; ++c) {
      const float alpha = __shfl_sync(0xffffffffu, my_a, c), bt = __shfl_sync(0xffffffffu, my_b, c);
      const float vt = col < dv ? __bfloat162float(v[static_cast<size_t>(tb + c) * vs + static_cast<size_t>(h) * dv + col]) : 0.f;
      float kv0 = 0.f, kv1 = 0.f, qs0 = 0.f, qs1 = 0.f;
#pragma unroll
      for (int i = 0; i < DK; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&s_k[c][i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&s_q[c][i]);
        kv0 += k4.x * S[i] + k4.z * S[i + 2];
        kv1 += k4.y * S[i + 1] + k4.w * S[i + 3];
        qs0 += q4.x * S[i] + q4.z * S[i + 2];
        qs1 += q4.y * S[i + 1] + q4.w * S[i + 3];
      }
      const float delta = bt * (vt - alpha * (kv0 + kv1));
      const float ot = alpha * (qs0 + qs1) + delta * s_qk[c];
#pragma unroll
      for (int i = 0; i < DK; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&s_k[c][i]);
        S[i] = fmaf(S[i], alpha, k4.x * delta);
        S[i + 1] = fmaf(S[i + 1], alpha, k4.y * delta);
        S[i + 2] = fmaf(S[i + 2], alpha, k4.z * delta);
        S[i + 3] = fmaf(S[i + 3], alpha, k4.w * delta);
      }
      if (col < dv) o[(static_cast<size_t>(tb + c) * Hv + h) * dv + col] = __float2bfloat16(ot);
    }
  }
  if (final_state != nullptr && col < dv) {
#pragma unroll
    for (int i = 0; i < DK; ++i) final_state[st_off + static_cast<size_t>(i) * dv] = S[i];
  }
}

// q, k [T, Hk, dk] and v [T, Hv, dv]: bf16 views with unit stride inside a head row and head stride dk / dv (token stride
// free, so slices of one fused projection are taken in place).  g, beta [T, Hv] fp32.  cu [n+1] int32.  init_state
// (optional) and the returned final state are [n, Hv, dk, dv] fp32.  Returns {o [T, Hv, dv] bf16, final_state}.
std::vector<torch::Tensor> gdn_recurrent_fwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, const torch::Tensor& g,
                                             const torch::Tensor& beta, const torch::Tensor& cu, const c10::optional<torch::Tensor>& init_state,
                                             double scale, bool want_state) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "q, k, v: [T, H, d]");
  for (const auto* t : {&q, &k, &v}) {
    TORCH_CHECK(t->scalar_type() == torch::kBFloat16 && t->stride(2) == 1 && t->stride(1) == t->size(2), "bf16 rows [H, d] contiguous per token");
  }
  const int T = q.size(0), Hk = q.size(1), dk = q.size(2), Hv = v.size(1), dv = v.size(2);
  TORCH_CHECK(k.size(0) == T && v.size(0) == T && k.size(1) == Hk && k.size(2) == dk, "q / k / v token and head counts");
  TORCH_CHECK(Hv % Hk == 0, "value heads must be a multiple of key heads");
  TORCH_CHECK(dk == 64 || dk == 128, "key head dim 64 or 128");
  TORCH_CHECK(g.scalar_type() == torch::kFloat32 && g.is_contiguous() && g.size(0) == T && g.size(1) == Hv, "g: [T, Hv] fp32");
  TORCH_CHECK(beta.scalar_type() == torch::kFloat32 && beta.is_contiguous() && beta.sizes() == g.sizes(), "beta: [T, Hv] fp32");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && cu.is_contiguous() && cu.numel() >= 1, "cu_seqlens int32");
  const int n_seq = cu.numel() - 1;
  c10::cuda::CUDAGuard guard(q.device());
  auto o = torch::empty({T, Hv, dv}, q.options());
  torch::Tensor fin = want_state ? torch::empty({n_seq, Hv, dk, dv}, q.options().dtype(torch::kFloat32)) : torch::Tensor();
  const float* init = nullptr;
  if (init_state.has_value() && init_state->defined()) {
    TORCH_CHECK(init_state->scalar_type() == torch::kFloat32 && init_state->is_contiguous() && init_state->numel() == static_cast<int64_t>(n_seq) * Hv * dk * dv,
                "init_state: [n, Hv, dk, dv] fp32");
    init = init_state->data_ptr<float>();
  }
  if (n_seq == 0 || (T == 0 && !want_state)) return {o, fin};
  TORCH_CHECK(n_seq <= 65535 && Hv <= 65535, "grid limits");
  dim3 grid((dv + 31) / 32, Hv, n_seq);
  auto stream = at::cuda::getCurrentCUDAStream();
  auto launch = [&](auto kern) {
    kern<<<grid, 32, 0, stream>>>(reinterpret_cast<const bf16*>(q.data_ptr()), reinterpret_cast<const bf16*>(k.data_ptr()),
                                  reinterpret_cast<const bf16*>(v.data_ptr()), q.stride(0), k.stride(0), v.stride(0), g.data_ptr<float>(),
                                  beta.data_ptr<float>(), cu.data_ptr<int>(), init, reinterpret_cast<bf16*>(o.data_ptr()),
                                  want_state ? fin.data_ptr<float>() : nullptr, Hv, Hv / Hk, dv, static_cast<float>(scale));
  };
  if (dk == 128) launch(gdn_recurrent_fwd_kernel<128>); else launch(gdn_recurrent_fwd_kernel<64>);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {o, fin};
}

}  // namespace tk
