// Token permutation kernels of the MoE block: dispatch (token rows → expert-grouped rows) and combine
// (expert-grouped rows → weighted sum per token).  Both directions are pure gathers — every destination row
// has exactly one writer — so there are no atomics and the result is deterministic:
//   rows_gather   : out[r] = scale[r] · x[src[r]]                 (src[r] < 0 → zero row)        dispatch fwd, combine bwd
//   rows_combine  : out[t] = Σ_j w[t,j] · y[row_of[t,j]]          (row_of < 0 → skipped)          combine fwd, dispatch bwd
//   combine_wgrad : dw[t,j] = <g[t], y[row_of[t,j]]>                                               router-weight gradient
// One warp per destination row; 16-byte accesses; bf16 data, fp32 math.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace tk {

using bf16 = __nv_bfloat16;

__global__ void __launch_bounds__(256) rows_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ src, const float* __restrict__ scale,
                                                           bf16* __restrict__ out, int R, int H) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int r = blockIdx.x * warps + (threadIdx.x >> 5); r < R; r += gridDim.x * warps) {
    const int s = src[r];
    uint4* o = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * H);
    if (s < 0) {
      for (int v = lane; v < nvec; v += 32) o[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* in = reinterpret_cast<const uint4*>(x + static_cast<size_t>(s) * H);
    if (scale == nullptr) {
      for (int v = lane; v < nvec; v += 32) o[v] = in[v];
    } else {
      const float c = scale[r];
      for (int v = lane; v < nvec; v += 32) {
        uint4 u = in[v];
        uint32_t* p = &u.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16(p[k]);
          p[k] = pack_bf16(f.x * c, f.y * c);
        }
        o[v] = u;
      }
    }
  }
}

template <int K>
__global__ void __launch_bounds__(256) rows_combine_kernel(const bf16* __restrict__ y, const int* __restrict__ row_of, const float* __restrict__ w,
                                                            bf16* __restrict__ out, int T, int H) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    int rows[K];
    float ws[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      rows[j] = row_of[static_cast<size_t>(t) * K + j];
      ws[j] = w ? w[static_cast<size_t>(t) * K + j] : 1.f;
    }
    uint4* o = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (rows[j] < 0) continue;
        const uint4 u = reinterpret_cast<const uint4*>(y + static_cast<size_t>(rows[j]) * H)[v];
        const uint32_t* p = &u.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16(p[k]);
          acc[2 * k] += ws[j] * f.x;
          acc[2 * k + 1] += ws[j] * f.y;
        }
      }
      o[v] = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
    }
  }
}

template <int K>
__global__ void __launch_bounds__(256) combine_wgrad_kernel(const bf16* __restrict__ g, const bf16* __restrict__ y, const int* __restrict__ row_of,
                                                             float* __restrict__ dw, int T, int H) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    float acc[K];
    int rows[K];
#pragma unroll
    for (int j = 0; j < K; ++j) { acc[j] = 0.f; rows[j] = row_of[static_cast<size_t>(t) * K + j]; }
    const uint4* gr = reinterpret_cast<const uint4*>(g + static_cast<size_t>(t) * H);
    for (int v = lane; v < nvec; v += 32) {
      const uint4 ug = gr[v];
      const uint32_t* pg = &ug.x;
      float gf[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) { const float2 f = unpack_bf16(pg[k]); gf[2 * k] = f.x; gf[2 * k + 1] = f.y; }
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (rows[j] < 0) continue;
        const uint4 u = reinterpret_cast<const uint4*>(y + static_cast<size_t>(rows[j]) * H)[v];
        const uint32_t* p = &u.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16(p[k]);
          acc[j] += gf[2 * k] * f.x + gf[2 * k + 1] * f.y;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const float s = warp_sum(acc[j]);
      if (lane == 0) dw[static_cast<size_t>(t) * K + j] = s;
    }
  }
}

static void check_rows(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.is_contiguous() && t.size(1) % 8 == 0, name,
              ": [rows, H] bf16 contiguous with H % 8 == 0");
}
static int grid_for(long rows) { return static_cast<int>(std::max<long>(1, std::min<long>((rows + 7) / 8, static_cast<long>(num_sms()) * 8))); }

torch::Tensor moe_rows_gather(const torch::Tensor& x, const torch::Tensor& src, const c10::optional<torch::Tensor>& scale) {
  check_rows(x, "x");
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == torch::kInt32 && src.is_contiguous(), "src int32");
  c10::cuda::CUDAGuard guard(x.device());
  const int R = src.numel(), H = x.size(1);
  auto out = torch::empty({R, H}, x.options());
  if (R == 0) return out;
  const float* sc = nullptr;
  if (scale.has_value() && scale->defined()) {
    TORCH_CHECK(scale->scalar_type() == torch::kFloat32 && scale->numel() == R && scale->is_contiguous(), "scale fp32 [R]");
    sc = scale->data_ptr<float>();
  }
  rows_gather_kernel<<<grid_for(R), 256, 0, at::cuda::getCurrentCUDAStream()>>>(reinterpret_cast<const bf16*>(x.data_ptr()), src.data_ptr<int>(), sc,
                                                                               reinterpret_cast<bf16*>(out.data_ptr()), R, H);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return out;
}

#define TK_K_SWITCH(K, BODY)                                   \
  switch (K) {                                                 \
    case 1: { constexpr int KK = 1; BODY; break; }             \
    case 2: { constexpr int KK = 2; BODY; break; }             \
    case 4: { constexpr int KK = 4; BODY; break; }             \
    case 6: { constexpr int KK = 6; BODY; break; }             \
    case 8: { constexpr int KK = 8; BODY; break; }             \
    default: TORCH_CHECK(false, "top-k must be 1, 2, 4, 6 or 8"); \
  }

torch::Tensor moe_rows_combine(const torch::Tensor& y, const torch::Tensor& row_of, const c10::optional<torch::Tensor>& w) {
  check_rows(y, "y");
  TORCH_CHECK(row_of.is_cuda() && row_of.scalar_type() == torch::kInt32 && row_of.dim() == 2 && row_of.is_contiguous(), "row_of int32 [T, k]");
  c10::cuda::CUDAGuard guard(y.device());
  const int T = row_of.size(0), K = row_of.size(1), H = y.size(1);
  auto out = torch::empty({T, H}, y.options());
  if (T == 0) return out;
  const float* wp = nullptr;
  if (w.has_value() && w->defined()) {
    TORCH_CHECK(w->scalar_type() == torch::kFloat32 && w->numel() == static_cast<int64_t>(T) * K && w->is_contiguous(), "w fp32 [T, k]");
    wp = w->data_ptr<float>();
  }
  auto stream = at::cuda::getCurrentCUDAStream();
  TK_K_SWITCH(K, (rows_combine_kernel<KK><<<grid_for(T), 256, 0, stream>>>(reinterpret_cast<const bf16*>(y.data_ptr()), row_of.data_ptr<int>(), wp,
                                                                           reinterpret_cast<bf16*>(out.data_ptr()), T, H)));
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return out;
}

torch::Tensor moe_combine_wgrad(const torch::Tensor& g, const torch::Tensor& y, const torch::Tensor& row_of) {
  check_rows(g, "g");
  check_rows(y, "y");
  TORCH_CHECK(row_of.scalar_type() == torch::kInt32 && row_of.dim() == 2 && row_of.is_contiguous() && row_of.size(0) == g.size(0), "row_of int32 [T, k]");
  TORCH_CHECK(g.size(1) == y.size(1), "H mismatch");
  c10::cuda::CUDAGuard guard(y.device());
  const int T = row_of.size(0), K = row_of.size(1), H = y.size(1);
  auto dw = torch::empty({T, K}, y.options().dtype(torch::kFloat32));
  if (T == 0) return dw;
  auto stream = at::cuda::getCurrentCUDAStream();
  TK_K_SWITCH(K, (combine_wgrad_kernel<KK><<<grid_for(T), 256, 0, stream>>>(reinterpret_cast<const bf16*>(g.data_ptr()), reinterpret_cast<const bf16*>(y.data_ptr()),
                                                                            row_of.data_ptr<int>(), dw.data_ptr<float>(), T, H)));
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return dw;
}

}  // namespace tk

// ------------------------------------------------------------------------------------------------------------
// Expert-parallel variants: the same gathers, but the source rows live in the symmetric buffers of the peer GPUs
// of the expert-parallel group and are read over NVLink from inside the kernel (plain peer loads).  The
// all-to-all "dispatch" is therefore fused with the regrouping into the 128-aligned expert layout, and the
// all-to-all "combine" with the weighted sum over the k experts of a token: no staging buffer, no NCCL call and no
// host-side split sizes.  Callers publish their buffers, pass one cross-GPU flag barrier, then launch these.
namespace tk {

constexpr int EP_MAX_PEERS = 8;
struct EpPtrs {
  const void* p[EP_MAX_PEERS];
};

// out[r] = scale · x_s[tok_s[pos]] with s = src_rank[r], pos = src_pos[r]; s < 0 → zero row.
// `total_rows` (device int) is checked against R once: rows that did not fit are reported through the error word.
// Every index that becomes a peer address is range-checked first (source rank against the group size, position against
// the capacity of the peers' token lists, token against the rows of the peers' activation buffers): a bad one records
// ERR_BOUNDS and yields a zero row instead of a wild NVLink read.  Once the error word is set (a peer never arrived at
// the barrier before this launch, or an earlier check failed) no peer memory is touched at all.
__global__ void __launch_bounds__(256) ep_rows_gather_kernel(EpPtrs xs, EpPtrs toks, EpPtrs ws, int use_w, const int* __restrict__ src_rank,
                                                              const int* __restrict__ src_pos, bf16* __restrict__ out, int R, int H,
                                                              const int* __restrict__ total_rows, int* err, int n_peers, int tok_cap, int x_rows) {
  if (*reinterpret_cast<volatile int*>(err) != 0) return;
  if (blockIdx.x == 0 && threadIdx.x == 0 && total_rows != nullptr && *total_rows > R) atomicCAS(err, 0, ERR_BOUNDS);
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  // rows past the last expert segment belong to no GEMM tile and are never read: leave them untouched
  const int used = total_rows != nullptr ? min(R, *total_rows) : R;
  for (int r = blockIdx.x * warps + (threadIdx.x >> 5); r < used; r += gridDim.x * warps) {
    const int s = src_rank[r];
    uint4* o = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * H);
    if (s < 0) {
      for (int v = lane; v < nvec; v += 32) o[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const int pos = src_pos[r];
    int tok = -1;
    if (s < n_peers && pos >= 0 && pos < tok_cap) tok = reinterpret_cast<const int*>(toks.p[s])[pos];
    if (tok < 0 || tok >= x_rows) {
      if (lane == 0) atomicCAS(err, 0, ERR_BOUNDS);
      for (int v = lane; v < nvec; v += 32) o[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const float c = use_w ? reinterpret_cast<const float*>(ws.p[s])[pos] : 1.f;
    const uint4* in = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(xs.p[s]) + static_cast<size_t>(tok) * H);
    for (int v = lane; v < nvec; v += 32) {
      uint4 u = in[v];
      if (use_w) {
        uint32_t* p = &u.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16(p[k]);
          p[k] = pack_bf16(f.x * c, f.y * c);
        }
      }
      o[v] = u;
    }
  }
}

// out[t] = Σ_j w[t,j] · y_{d}[row] with d = dst_rank[t,j] (< 0 → skipped), row = dst_row[t,j].
template <int K>
__global__ void __launch_bounds__(256) ep_rows_combine_kernel(EpPtrs ys, const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                                                               const float* __restrict__ w, bf16* __restrict__ out, int T, int H, int* err,
                                                               int n_peers, int y_rows) {
  if (*reinterpret_cast<volatile int*>(err) != 0) return;
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    const uint4* src[K];
    float ws[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int d = dst_rank[static_cast<size_t>(t) * K + j];
      const int row = dst_row[static_cast<size_t>(t) * K + j];
      const bool bad = d >= n_peers || (d >= 0 && (row < 0 || row >= y_rows));
      if (bad && lane == 0) atomicCAS(err, 0, ERR_BOUNDS);
      src[j] = (d < 0 || bad) ? nullptr : reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(ys.p[d]) + static_cast<size_t>(row) * H);
      ws[j] = w ? w[static_cast<size_t>(t) * K + j] : 1.f;
    }
    uint4* o = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (src[j] == nullptr) continue;
        const uint4 u = src[j][v];
        const uint32_t* p = &u.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16(p[k]);
          acc[2 * k] += ws[j] * f.x;
          acc[2 * k + 1] += ws[j] * f.y;
        }
      }
      o[v] = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
    }
  }
}

// dw[t,j] = <g[t], y_{d}[row]>
template <int K>
__global__ void __launch_bounds__(256) ep_combine_wgrad_kernel(const bf16* __restrict__ g, EpPtrs ys, const int* __restrict__ dst_rank,
                                                                const int* __restrict__ dst_row, float* __restrict__ dw, int T, int H, int* err,
                                                                int n_peers, int y_rows) {
  if (*reinterpret_cast<volatile int*>(err) != 0) return;
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps) {
    const uint4* src[K];
    float acc[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int d = dst_rank[static_cast<size_t>(t) * K + j];
      const int row = dst_row[static_cast<size_t>(t) * K + j];
      const bool bad = d >= n_peers || (d >= 0 && (row < 0 || row >= y_rows));
      if (bad && lane == 0) atomicCAS(err, 0, ERR_BOUNDS);
      src[j] = (d < 0 || bad) ? nullptr : reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(ys.p[d]) + static_cast<size_t>(row) * H);
      acc[j] = 0.f;
    }
    const uint4* gr = reinterpret_cast<const uint4*>(g + static_cast<size_t>(t) * H);
    for (int v = lane; v < nvec; v += 32) {
      const uint4 ug = gr[v];
      const uint32_t* pg = &ug.x;
      float gf[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) { const float2 f = unpack_bf16(pg[k]); gf[2 * k] = f.x; gf[2 * k + 1] = f.y; }
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (src[j] == nullptr) continue;
        const uint4 u = src[j][v];
        const uint32_t* p = &u.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16(p[k]);
          acc[j] += gf[2 * k] * f.x + gf[2 * k + 1] * f.y;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const float s = warp_sum(acc[j]);
      if (lane == 0) dw[static_cast<size_t>(t) * K + j] = s;
    }
  }
}

static EpPtrs to_ptrs(const std::vector<int64_t>& v) {
  TORCH_CHECK(v.size() <= EP_MAX_PEERS, "expert-parallel group larger than ", EP_MAX_PEERS);
  EpPtrs p{};
  for (size_t i = 0; i < v.size(); ++i) p.p[i] = reinterpret_cast<const void*>(v[i]);
  return p;
}
static void check_i32(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous(), name, " must be a contiguous int32 CUDA tensor");
}

// `tok_cap`: entries of every peer's token (and weight) list; `x_rows`: rows of every peer's activation buffer.
torch::Tensor ep_rows_gather(const std::vector<int64_t>& x_ptrs, const std::vector<int64_t>& tok_ptrs, const std::vector<int64_t>& w_ptrs,
                             const torch::Tensor& src_rank, const torch::Tensor& src_pos, int64_t H, const torch::Tensor& total_rows,
                             int64_t tok_cap, int64_t x_rows) {
  TORCH_CHECK(tok_cap > 0 && x_rows > 0 && tok_ptrs.size() == x_ptrs.size(), "ep_rows_gather: capacities of the peers' buffers are required");
  check_i32(src_rank, "src_rank");
  check_i32(src_pos, "src_pos");
  check_i32(total_rows, "total_rows");
  TORCH_CHECK(H % 8 == 0 && src_rank.numel() == src_pos.numel(), "bad shapes");
  c10::cuda::CUDAGuard guard(src_rank.device());
  const int R = src_rank.numel();
  auto out = torch::empty({R, H}, src_rank.options().dtype(torch::kBFloat16));
  if (R == 0) return out;
  ep_rows_gather_kernel<<<grid_for(R), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      to_ptrs(x_ptrs), to_ptrs(tok_ptrs), to_ptrs(w_ptrs), w_ptrs.empty() ? 0 : 1, src_rank.data_ptr<int>(), src_pos.data_ptr<int>(),
      reinterpret_cast<bf16*>(out.data_ptr()), R, static_cast<int>(H), total_rows.data_ptr<int>(), error_word(), static_cast<int>(x_ptrs.size()),
      static_cast<int>(tok_cap), static_cast<int>(x_rows));
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return out;
}

torch::Tensor ep_rows_combine(const std::vector<int64_t>& y_ptrs, const torch::Tensor& dst_rank, const torch::Tensor& dst_row,
                              const c10::optional<torch::Tensor>& w, int64_t H, int64_t y_rows) {
  TORCH_CHECK(y_rows > 0, "ep_rows_combine: the row capacity of the peers' buffers is required");
  check_i32(dst_rank, "dst_rank");
  check_i32(dst_row, "dst_row");
  TORCH_CHECK(dst_rank.dim() == 2 && dst_row.sizes() == dst_rank.sizes() && H % 8 == 0, "bad shapes");
  c10::cuda::CUDAGuard guard(dst_rank.device());
  const int T = dst_rank.size(0), K = dst_rank.size(1);
  auto out = torch::empty({T, H}, dst_rank.options().dtype(torch::kBFloat16));
  if (T == 0) return out;
  const float* wp = nullptr;
  if (w.has_value() && w->defined()) {
    TORCH_CHECK(w->scalar_type() == torch::kFloat32 && w->is_contiguous() && w->numel() == static_cast<int64_t>(T) * K, "w fp32 [T, k]");
    wp = w->data_ptr<float>();
  }
  auto stream = at::cuda::getCurrentCUDAStream();
  const EpPtrs ys = to_ptrs(y_ptrs);
  TK_K_SWITCH(K, (ep_rows_combine_kernel<KK><<<grid_for(T), 256, 0, stream>>>(ys, dst_rank.data_ptr<int>(), dst_row.data_ptr<int>(), wp,
                                                                              reinterpret_cast<bf16*>(out.data_ptr()), T, static_cast<int>(H), error_word(),
                                                                              static_cast<int>(y_ptrs.size()), static_cast<int>(y_rows))));
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return out;
}

torch::Tensor ep_combine_wgrad(const torch::Tensor& g, const std::vector<int64_t>& y_ptrs, const torch::Tensor& dst_rank, const torch::Tensor& dst_row,
                               int64_t y_rows) {
  TORCH_CHECK(y_rows > 0, "ep_combine_wgrad: the row capacity of the peers' buffers is required");
  check_rows(g, "g");
  check_i32(dst_rank, "dst_rank");
  check_i32(dst_row, "dst_row");
  c10::cuda::CUDAGuard guard(g.device());
  const int T = dst_rank.size(0), K = dst_rank.size(1), H = g.size(1);
  TORCH_CHECK(g.size(0) == T, "row mismatch");
  auto dw = torch::empty({T, K}, g.options().dtype(torch::kFloat32));
  if (T == 0) return dw;
  auto stream = at::cuda::getCurrentCUDAStream();
  const EpPtrs ys = to_ptrs(y_ptrs);
  TK_K_SWITCH(K, (ep_combine_wgrad_kernel<KK><<<grid_for(T), 256, 0, stream>>>(reinterpret_cast<const bf16*>(g.data_ptr()), ys, dst_rank.data_ptr<int>(),
                                                                               dst_row.data_ptr<int>(), dw.data_ptr<float>(), T, H, error_word(),
                                                                               static_cast<int>(y_ptrs.size()), static_cast<int>(y_rows))));
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return dw;
}

}  // namespace tk
