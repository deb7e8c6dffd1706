// Sampler kernels: paged-KV decode attention (one query token per sequence, GQA), token sampling
// (temperature / top-k / top-p via threshold bisection + Gumbel-max, log-prob of the processed
// distribution), and the MoE router (fp32 softmax + top-k + renormalisation + expert histogram).
// All three are bandwidth / latency bound; none needs tensor cores.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace tk {

using bf16 = __nv_bfloat16;

// ---------------------------------------------------------------- paged decode
// One CTA per (sequence, kv head, group of GH query heads); 4 warps.  A warp handles 4 context tokens per step —
// 8 lanes per token, 16 dims (two 16-byte loads of K, two of V) per lane — and two steps are issued back to back, so
// 32 token rows per CTA are in flight.  Every lane group keeps an online-softmax state per query head; lane groups
// and warps are merged at the end.
template <int GH>
__global__ void __launch_bounds__(128) paged_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                                                            const int* __restrict__ tables, const int* __restrict__ seq_lens, bf16* __restrict__ out,
                                                            int hq, int hkv, int block_size, int max_blocks, float scale_log2, int G) {
  constexpr int D = 128;
  const int b = blockIdx.x, kvh = blockIdx.y, h0 = kvh * G + blockIdx.z * GH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane >> 3, sub = lane & 7;  // sub owns dims [16·sub, 16·sub+16)
  const int n = seq_lens[b];
  // the query (pre-scaled, fp32) lives in shared memory: registers are kept for two iterations' worth of K/V rows
  __shared__ float s_q[GH][D];
  for (int i = threadIdx.x; i < GH * D; i += blockDim.x)
    s_q[i / D][i % D] = __bfloat162float(q[(static_cast<size_t>(b) * hq + h0 + i / D) * D + i % D]) * scale_log2;
  __syncthreads();
  float m[GH], l[GH], acc[GH][16];
#pragma unroll
  for (int g = 0; g < GH; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < 16; ++d) acc[g][d] = 0.f;
  }
  const int* table = tables + static_cast<size_t>(b) * max_blocks;
  // token handled by (warp, grp) in half-step u of iteration `base`: t = base + grp + 16·u.  The loop bound depends on
  // the warp only, so all 32 lanes stay in the loop together (the shuffles below name the full warp).  The rows of
  // iteration i+1 are requested before iteration i is consumed.
  uint4 kr[2][2], vr[2][2], kn[2][2], vn[2][2];
  auto fetch = [&](int base, uint4 (&kk)[2][2], uint4 (&vv)[2][2]) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int t = base + grp + u * 16;
      if (t < n) {
        const int blk = table[t / block_size], off = t % block_size;
        // lane `sub` owns dims [8·sub, 8·sub+8) and [64+8·sub, 64+8·sub+8): each load instruction covers 128 contiguous bytes per token
        const size_t base_off = ((static_cast<size_t>(blk) * block_size + off) * hkv + kvh) * D + sub * 8;
        kk[u][0] = *reinterpret_cast<const uint4*>(kc + base_off); kk[u][1] = *reinterpret_cast<const uint4*>(kc + base_off + 64);
        vv[u][0] = *reinterpret_cast<const uint4*>(vc + base_off); vv[u][1] = *reinterpret_cast<const uint4*>(vc + base_off + 64);
      }
    }
  };
  if (warp * 4 < n) fetch(warp * 4, kr, vr);
  for (int base = warp * 4; base < n; base += 32) {
    if (base + 32 < n) fetch(base + 32, kn, vn);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const bool live = base + grp + u * 16 < n;
      float kf[16], vf[16];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t* pk = &kr[u][h].x;
        const uint32_t* pv = &vr[u][h].x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 a = unpack_bf16(pk[k]), c = unpack_bf16(pv[k]);
          kf[h * 8 + 2 * k] = a.x; kf[h * 8 + 2 * k + 1] = a.y;
          vf[h * 8 + 2 * k] = c.x; vf[h * 8 + 2 * k + 1] = c.y;
        }
      }
#pragma unroll
      for (int g = 0; g < GH; ++g) {
        float s = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float4* qs = reinterpret_cast<const float4*>(&s_q[g][h * 64 + sub * 8]);
#pragma unroll
          for (int d4 = 0; d4 < 2; ++d4) {
            const float4 qq = qs[d4];
            s += qq.x * kf[h * 8 + 4 * d4] + qq.y * kf[h * 8 + 4 * d4 + 1] + qq.z * kf[h * 8 + 4 * d4 + 2] + qq.w * kf[h * 8 + 4 * d4 + 3];
          }
        }
        if (!live) s = 0.f;  // rows that were not fetched hold stale registers
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (live) {  // uniform inside an 8-lane group
          const float mn = fmaxf(m[g], s);
          const float corr = exp2f(m[g] - mn), p = exp2f(s - mn);
          l[g] = l[g] * corr + p;
#pragma unroll
          for (int d = 0; d < 16; ++d) acc[g][d] = acc[g][d] * corr + p * vf[d];
          m[g] = mn;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      kr[u][0] = kn[u][0]; kr[u][1] = kn[u][1];
      vr[u][0] = vn[u][0]; vr[u][1] = vn[u][1];
    }
  }
  // merge the 4 lane groups of the warp, then the 4 warps
  __shared__ float s_m[4][GH], s_l[4][GH], s_acc[4][GH][D];
#pragma unroll
  for (int g = 0; g < GH; ++g) {
#pragma unroll
    for (int o = 8; o <= 16; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o), lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], mo);
      const float c0 = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn), c1 = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
#pragma unroll
      for (int d = 0; d < 16; ++d) acc[g][d] = acc[g][d] * c0 + __shfl_xor_sync(0xffffffffu, acc[g][d], o) * c1;
      l[g] = l[g] * c0 + lo * c1;
      m[g] = mn;
    }
    if (lane == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
    if (grp == 0) {
#pragma unroll
      for (int d = 0; d < 16; ++d) s_acc[warp][g][(d >> 3) * 64 + sub * 8 + (d & 7)] = acc[g][d];
    }
  }
  __syncthreads();
  const int d = threadIdx.x;  // thread d (0..127) finishes dimension d of every head of the group
#pragma unroll
  for (int g = 0; g < GH; ++g) {
    const float mm = fmaxf(fmaxf(s_m[0][g], s_m[1][g]), fmaxf(s_m[2][g], s_m[3][g]));
    float ll = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = (s_m[w][g] == -INFINITY) ? 0.f : exp2f(s_m[w][g] - mm);
      ll += s_l[w][g] * c;
      o += s_acc[w][g][d] * c;
    }
    out[(static_cast<size_t>(b) * hq + h0 + g) * D + d] = __float2bfloat16(ll > 0.f ? o / ll : 0.f);
  }
}

torch::Tensor paged_attn_decode(const torch::Tensor& q, const torch::Tensor& kc, const torch::Tensor& vc, const torch::Tensor& tables,
                                const torch::Tensor& seq_lens, double scale) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == torch::kBFloat16 && q.is_contiguous() && q.dim() == 3 && q.size(2) == 128, "q [B,Hq,128] bf16");
  TORCH_CHECK(kc.is_contiguous() && vc.is_contiguous() && kc.dim() == 4 && kc.size(3) == 128 && kc.scalar_type() == torch::kBFloat16, "cache [blocks,bs,Hkv,128] bf16");
  TORCH_CHECK(tables.scalar_type() == torch::kInt32 && tables.is_contiguous() && seq_lens.scalar_type() == torch::kInt32, "int32 tables / lens");
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), hq = q.size(1), hkv = kc.size(2), G = hq / hkv;
  auto out = torch::empty_like(q);
  if (B == 0) return out;
  const float sl2 = static_cast<float>(scale * 1.4426950408889634);
  auto stream = at::cuda::getCurrentCUDAStream();
  // query heads of a group are processed GH at a time (register budget): G = 8 → two CTAs per (sequence, kv head)
  const int GH = G >= 4 ? 4 : G;
  TORCH_CHECK(G == 1 || G == 2 || G == 4 || G == 8, "GQA group size must be 1, 2, 4 or 8");
  dim3 grid(B, hkv, G / GH);
#define TK_DEC(GG)                                                                                                                   \
  paged_decode_kernel<GG><<<grid, 128, 0, stream>>>(reinterpret_cast<const bf16*>(q.data_ptr()), reinterpret_cast<const bf16*>(kc.data_ptr()), \
      reinterpret_cast<const bf16*>(vc.data_ptr()), tables.data_ptr<int>(), seq_lens.data_ptr<int>(), reinterpret_cast<bf16*>(out.data_ptr()),  \
      hq, hkv, static_cast<int>(kc.size(1)), static_cast<int>(tables.size(1)), sl2, G)
  switch (GH) {
    case 1: TK_DEC(1); break;
    case 2: TK_DEC(2); break;
    default: TK_DEC(4); break;
  }
#undef TK_DEC
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return out;
}

// -------------------------------------------------------------------- sampling
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float r = lane < nw ? sh[lane] : (is_max ? -INFINITY : 0.f);
  r = is_max ? warp_max(r) : warp_sum(r);
  return __shfl_sync(0xffffffffu, r, 0);
}
__device__ __forceinline__ uint32_t mix32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
  return static_cast<uint32_t>(x);
}

// One CTA per row.  kept set = {p ≥ τ}: τ from bisection so that |kept| ≤ top_k-ish and mass(kept) ≥ top_p
// (the smallest such set up to ties).  Token = argmax over kept of (x/T + Gumbel noise).
__global__ void __launch_bounds__(512) sample_kernel(const float* __restrict__ logits, const int64_t* __restrict__ seeds, int64_t* __restrict__ tok,
                                                      float* __restrict__ logprob, int V, float inv_temp, int top_k, float top_p, int greedy) {
  __shared__ float sh[32];
  __shared__ int sh_i[32];
  const int row = blockIdx.x;
  const float* x = logits + static_cast<size_t>(row) * V;
  // max and sum-exp in one pass (online softmax per thread, merged across the block)
  float mx = -INFINITY, z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float y = x[i] * inv_temp;
    if (y > mx) { z = z * __expf(mx - y) + 1.f; mx = y; } else { z += __expf(y - mx); }
  }
  {
    const float m_all = block_reduce(mx, true, sh);
    z = block_reduce(z * __expf(mx - m_all), false, sh);
    mx = m_all;
  }
  float tau = 0.f, kept_mass = 1.f;  // threshold on p = e^{x−mx}/z
  const bool use_k = top_k > 0 && top_k < V, use_p = top_p < 1.f;
  if (!greedy && (use_k || use_p)) {
    // τ_k: highest threshold that still keeps ≥ k tokens; τ_p: highest that still keeps mass ≥ top_p; the kept set
    // respects both limits → τ = max(τ_k, τ_p).  Each pass over the row tests 15 thresholds per search (16-way
    // narrowing of [lo, hi)), so 8 passes resolve both thresholds to 2⁻³² of the largest probability.
    constexpr int NT = 15;
    float lo_k = 0.f, hi_k = 1.f / z, lo_p = 0.f, hi_p = 1.f / z;  // p_max = 1/z
    const float inv_z = 1.f / z;
    for (int it = 0; it < 8; ++it) {
      float ck[NT], cp[NT];
#pragma unroll
      for (int j = 0; j < NT; ++j) { ck[j] = 0.f; cp[j] = 0.f; }
      const float dk = (hi_k - lo_k) * (1.f / 16.f), dp = (hi_p - lo_p) * (1.f / 16.f);
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float p = __expf(x[i] * inv_temp - mx) * inv_z;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          ck[j] += (p >= lo_k + dk * (j + 1)) ? 1.f : 0.f;
          cp[j] += (p >= lo_p + dp * (j + 1)) ? p : 0.f;
        }
      }
      int jk = -1, jp = -1;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const float a_k = use_k ? block_reduce(ck[j], false, sh) : 0.f;
        const float a_p = use_p ? block_reduce(cp[j], false, sh) : 0.f;
        if (a_k >= static_cast<float>(top_k)) jk = j;   // counts and masses fall with j: the last j that passes is the highest
        if (a_p >= top_p) jp = j;
      }
      const float nlo_k = lo_k + dk * (jk + 1), nlo_p = lo_p + dp * (jp + 1);
      hi_k = (jk == NT - 1) ? hi_k : nlo_k + dk;
      hi_p = (jp == NT - 1) ? hi_p : nlo_p + dp;
      lo_k = nlo_k;
      lo_p = nlo_p;
    }
    tau = fmaxf(use_k ? lo_k : 0.f, use_p ? lo_p : 0.f);
    float mass = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float p = __expf(x[i] * inv_temp - mx) * inv_z;
      if (p >= tau) mass += p;
    }
    kept_mass = block_reduce(mass, false, sh);
  }
  float best = -INFINITY;
  int best_i = 0;
  const uint64_t seed = static_cast<uint64_t>(seeds[row]);
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float xs = x[i] * inv_temp;
    const float p = __expf(xs - mx) / z;
    if (p < tau) continue;
    float score = xs;
    if (!greedy) {
      const float u = (static_cast<float>(mix32(seed * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(i))) + 0.5f) * (1.f / 4294967296.f);
      score += -__logf(-__logf(u));
    }
    if (score > best) { best = score; best_i = i; }
  }
  // block arg-max
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) { sh[warp] = best; sh_i[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? sh[lane] : -INFINITY;
    best_i = lane < (blockDim.x >> 5) ? sh_i[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
    }
    if (lane == 0) {
      tok[row] = best_i;
      logprob[row] = greedy ? 0.f : (x[best_i] * inv_temp - mx - __logf(z) - __logf(kept_mass));
    }
  }
}

std::vector<torch::Tensor> sample_tokens(const torch::Tensor& logits, double temperature, int64_t top_k, double top_p, const torch::Tensor& seeds) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == torch::kFloat32 && logits.is_contiguous() && logits.dim() == 2, "logits [B,V] fp32");
  TORCH_CHECK(seeds.is_cuda() && seeds.scalar_type() == torch::kInt64 && seeds.numel() == logits.size(0), "seeds int64 [B]");
  c10::cuda::CUDAGuard guard(logits.device());
  const int B = logits.size(0), V = logits.size(1);
  auto tok = torch::empty({B}, logits.options().dtype(torch::kInt64));
  auto lp = torch::empty({B}, logits.options());
  if (B == 0) return {tok, lp};
  const bool greedy = temperature <= 0.0;
  sample_kernel<<<B, 512, 0, at::cuda::getCurrentCUDAStream()>>>(logits.data_ptr<float>(), seeds.data_ptr<int64_t>(), tok.data_ptr<int64_t>(),
                                                                 lp.data_ptr<float>(), V, greedy ? 1.f : static_cast<float>(1.0 / temperature),
                                                                 static_cast<int>(top_k), static_cast<float>(top_p), greedy ? 1 : 0);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {tok, lp};
}

// ---------------------------------------------------------------------- router
// One warp per token, E ≤ 256 experts (≤ 8 per lane).  Outputs probs [T,E] fp32, top-k weights (optionally
// renormalised) and indices, and adds to the per-expert histogram.
template <int PER_LANE>
__global__ void moe_router_kernel(const bf16* __restrict__ logits_bf, const float* __restrict__ logits_f, float* __restrict__ probs,
                                  float* __restrict__ weights, int64_t* __restrict__ indices, int* __restrict__ hist, int T, int E, int k,
                                  int renorm) {
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < T; t += gridDim.x * (blockDim.x >> 5)) {
    float v[PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      const int e = j * 32 + lane;
      v[j] = e < E ? (logits_f ? logits_f[static_cast<size_t>(t) * E + e] : __bfloat162float(logits_bf[static_cast<size_t>(t) * E + e])) : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float z = 0.f;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) { v[j] = (j * 32 + lane < E) ? __expf(v[j] - mx) : 0.f; z += v[j]; }
    z = warp_sum(z);
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      v[j] /= z;
      if (j * 32 + lane < E) probs[static_cast<size_t>(t) * E + j * 32 + lane] = v[j];
    }
    float sel_sum = 0.f, my_w = 0.f;
    int my_i = 0;
    for (int r = 0; r < k; ++r) {
      float best = -1.f;
      int bi = 0;
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j) if (v[j] > best) { best = v[j]; bi = j * 32 + lane; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if ((bi & 31) == lane) v[bi >> 5] = -2.f;  // remove the winner
      sel_sum += best;
      if (lane == r) { my_w = best; my_i = bi; }
    }
    if (lane < k) {
      weights[static_cast<size_t>(t) * k + lane] = renorm ? my_w / sel_sum : my_w;
      indices[static_cast<size_t>(t) * k + lane] = my_i;
      if (hist) atomicAdd(&hist[my_i], 1);
    }
  }
}

std::vector<torch::Tensor> moe_router(const torch::Tensor& logits, int64_t k, bool renorm) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous(), "logits [T,E]");
  const int T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(E <= 256 && k <= 32 && k <= E, "router supports up to 256 experts and top-32");
  c10::cuda::CUDAGuard guard(logits.device());
  auto f32 = logits.options().dtype(torch::kFloat32);
  auto probs = torch::empty({T, E}, f32);
  auto w = torch::empty({T, k}, f32);
  auto idx = torch::empty({T, k}, logits.options().dtype(torch::kInt64));
  auto hist = torch::zeros({E}, logits.options().dtype(torch::kInt32));
  if (T == 0) return {w, idx, probs, hist};
  const bf16* lb = logits.scalar_type() == torch::kBFloat16 ? reinterpret_cast<const bf16*>(logits.data_ptr()) : nullptr;
  const float* lf = logits.scalar_type() == torch::kFloat32 ? logits.data_ptr<float>() : nullptr;
  TORCH_CHECK(lb || lf, "router logits must be bf16 or fp32");
  const int blocks = std::min((T + 7) / 8, num_sms() * 8);
  auto stream = at::cuda::getCurrentCUDAStream();
#define TK_ROUTER(PL) moe_router_kernel<PL><<<blocks, 256, 0, stream>>>(lb, lf, probs.data_ptr<float>(), w.data_ptr<float>(), idx.data_ptr<int64_t>(), \
                                                                         hist.data_ptr<int>(), T, E, static_cast<int>(k), renorm ? 1 : 0)
  if (E <= 32) TK_ROUTER(1); else if (E <= 64) TK_ROUTER(2); else if (E <= 128) TK_ROUTER(4); else TK_ROUTER(8);
#undef TK_ROUTER
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {w, idx, probs, hist};
}

}  // namespace tk
