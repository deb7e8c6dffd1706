// bf16 GEMM on 5th-generation tensor cores (tcgen05) for sm_100a.
//
//   D[M,N] (+)= A · B with fp32 accumulation in tensor memory.
//   Layouts (all row-major tensors in global memory):
//     NT : A[M,K], B[N,K]   (both K-major)          forward  y = x Wᵀ
//     NN : A[M,K], B[K,N]   (B MN-major)            dgrad    dx = dy W
//     TN : A[K,M], B[K,N]   (both MN-major)         wgrad    dW = dyᵀ x
//
// Structure: persistent CTAs (one per SM), 192 threads:
//   warp 0      TMA producer   (cp.async.bulk.tensor 2-D, 128-byte swizzle, 4-stage mbarrier ring)
//   warp 1      MMA issuer     (one elected thread issues tcgen05.mma 128x256x16, commits to mbarriers)
//   warps 2..5  epilogue       (tcgen05.ld 32x32b → registers → bf16/fp32 global stores)
// The 512 TMEM columns hold two 128x256 fp32 accumulators so the epilogue of
// tile i overlaps the main loop of tile i+1.  Grouped (per-expert) variants
// share the same pipeline and differ only in the tile scheduler.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "host.h"

namespace tk {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int GROUP_M = 16;

struct GemmParams {
  void* out;       // bf16 or fp32
  int M, N, K;
  int ldo;         // leading dimension of out (elements)
  int out_fp32;    // 1: fp32 output
  int accumulate;  // 1: out += result
  int* err;
  // grouped mode
  const int* offsets;  // [E+1] row offsets (aligned to BM) or nullptr
  int num_groups;
  int group_rows_b;    // rows of B per group (N for NT, K for NN)
  int mode;            // 0 dense, 1 grouped over M (A rows by expert), 2 grouped wgrad (K range by expert)
  const int* group_map;  // optional: group g uses weight block group_map[g] (< 0: group skipped); nullptr = identity
  // second operand pair of the M-grouped mode (0 = none): out = A·B + A2·B2 accumulated in tensor memory before the
  // epilogue — how a low-rank (LoRA) term rides in the base GEMM instead of re-reading and re-writing the output
  int K2;
  int group_rows_b2;   // rows of B2 per group (N for NT, K2 for NN)
};

struct TileCoord {
  int m0, n0, group, k_begin, k_end, m_limit;
};

// Dense schedule: tiles are numbered so that GROUP_M consecutive M-tiles share each N-tile
// (the concurrently running CTAs then touch ~equal numbers of A and B rows → best L2 reuse).
__device__ __forceinline__ bool dense_tile(const GemmParams& p, int tile, TileCoord& t) {
  int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  if (tile >= num_m * num_n) return false;
  int per_group = GROUP_M * num_n;
  int g = tile / per_group, first_m = g * GROUP_M;
  int gsize = min(num_m - first_m, GROUP_M);
  int r = tile - g * per_group;
  t.m0 = (first_m + r % gsize) * BM;
  t.n0 = (r / gsize) * BN;
  t.group = 0;
  t.k_begin = 0;
  t.k_end = p.K;
  t.m_limit = p.M;
  return true;
}

// Grouped over M: each expert owns rows [offsets[e], offsets[e+1]) of A and of the output, and its own B.
struct GroupedCursor {
  int e = 0, tiles_before = 0;
};
__device__ __forceinline__ bool grouped_m_tile(const GemmParams& p, int tile, GroupedCursor& c, TileCoord& t) {
  int num_n = (p.N + BN - 1) / BN;
  while (c.e < p.num_groups) {
    int rows = p.offsets[c.e + 1] - p.offsets[c.e];
    if (p.group_map != nullptr && p.group_map[c.e] < 0) rows = 0;
    int tiles_e = ((rows + BM - 1) / BM) * num_n;
    if (tile < c.tiles_before + tiles_e) {
      int r = tile - c.tiles_before;
      int num_m = (rows + BM - 1) / BM;
      t.m0 = p.offsets[c.e] + (r % num_m) * BM;
      t.n0 = (r / num_m) * BN;
      t.group = c.e;
      t.k_begin = 0;
      t.k_end = p.K;
      t.m_limit = p.offsets[c.e + 1];
      return true;
    }
    c.tiles_before += tiles_e;
    ++c.e;
  }
  return false;
}
// Grouped wgrad: output [E, M, N]; expert e reduces over token rows [offsets[e], offsets[e+1]).
__device__ __forceinline__ bool grouped_k_tile(const GemmParams& p, int tile, TileCoord& t) {
  int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  int per_e = num_m * num_n;
  if (tile >= per_e * p.num_groups) return false;
  int e = tile / per_e, r = tile - e * per_e;
  t.m0 = (r % num_m) * BM;
  t.n0 = (r / num_m) * BN;
  t.group = e;
  t.k_begin = p.offsets[e];
  t.k_end = p.offsets[e + 1];
  t.m_limit = p.M;
  return true;
}

template <int MODE>
__device__ __forceinline__ bool next_tile(const GemmParams& p, int tile, GroupedCursor& c, TileCoord& t) {
  if constexpr (MODE == 0) return dense_tile(p, tile, t);
  else if constexpr (MODE == 1) return grouped_m_tile(p, tile, c, t);
  else return grouped_k_tile(p, tile, t);
}

template <bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      GroupedCursor cur;
      TileCoord t;
      bool ok = true;
      for (int tile = blockIdx.x; ok && next_tile<MODE>(p, tile, cur, t); tile += gridDim.x) {
        const int b_group = (MODE == 1) ? (p.group_map ? p.group_map[t.group] : t.group) : 0;
        const int b_row0 = b_group * p.group_rows_b;
        auto load_stage = [&](const CUtensorMap* mA, const CUtensorMap* mB, int k0, int brow) -> bool {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.err, ERR_PRODUCER_WAIT)) return false;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(sa, mA, &full_bar[stage], k0, t.m0);            // box {64 (K), 128 rows}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)                             // box {64 (M), 64 K-rows} each
              tma_load_2d(sa + j * (64 * BK * 2), mA, &full_bar[stage], t.m0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, mB, &full_bar[stage], k0, brow + t.n0);   // box {64 (K), 256 rows}
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), mB, &full_bar[stage], t.n0 + j * 64, brow + k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          return true;
        };
        for (int k0 = t.k_begin; ok && k0 < t.k_end; k0 += BK) ok = load_stage(&tmA, &tmB, k0, b_row0);
        if constexpr (MODE == 1) {
          // second pair: columns past K2 and rows past the tensors read as zero (out-of-range fill), so a K2 below the
          // 64-wide k-tile costs one tile
          for (int k0 = 0; ok && k0 < p.K2; k0 += BK) ok = load_stage(&tmA2, &tmB2, k0, b_group * p.group_rows_b2);
        }
      }
      if (!ok) {
        // drain: give in-flight copies a bounded chance to land before the CTA exits
        for (int s = 0; s < STAGES; ++s) mbar_wait(&full_bar[s], 0, nullptr, 0);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0, acc = 0, acc_phase = 0;
      GroupedCursor cur;
      TileCoord t;
      bool ok = true;
      for (int tile = blockIdx.x; ok && next_tile<MODE>(p, tile, cur, t); tile += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.err, ERR_MMA_WAIT_TMEM)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t first = 1;
        if (t.k_end <= t.k_begin) {
          // empty reduction range (expert without tokens): accumulator must read as zero → epilogue handles via flag
        }
        int k_tiles = (t.k_end > t.k_begin) ? (t.k_end - t.k_begin + BK - 1) / BK : 0;
        if constexpr (MODE == 1) k_tiles += (p.K2 + BK - 1) / BK;
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!mbar_wait(&full_bar[stage], phase, p.err, ERR_MMA_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad = A_MN ? umma_desc(sa + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                               : umma_desc(sa + k * (UMMA_K * 2), 16, 1024);
            uint64_t bd = B_MN ? umma_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                               : umma_desc(sb + k * (UMMA_K * 2), 16, 1024);
            umma_bf16(d_tmem, ad, bd, idesc, first ? 0u : 1u);
            first = 0;
          }
          umma_commit(&empty_bar[stage]);  // frees this smem stage once the MMAs above retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&tmem_full[acc]);      // accumulator complete → epilogue
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t acc = 0, acc_phase = 0;
    GroupedCursor cur;
    TileCoord t;
    bool ok = true;
    for (int tile = blockIdx.x; ok && next_tile<MODE>(p, tile, cur, t); tile += gridDim.x) {
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.err, ERR_EPI_WAIT)) { ok = false; break; }
      tc_fence_after();
      const bool empty_k = (t.k_end <= t.k_begin) && !(MODE == 1 && p.K2 > 0);
      const int row = t.m0 + q * 32 + lane;
      const bool row_ok = row < t.m_limit;
      size_t out_row = static_cast<size_t>(row);
      if constexpr (MODE == 2) out_row += static_cast<size_t>(t.group) * p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = t.n0 + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        if (empty_k) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (p.out_fp32) {
          float* o = reinterpret_cast<float*>(p.out) + out_row * p.ldo + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (col0 + j + 4 <= p.N) {
              float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                     __uint_as_float(r[j + 3]));
              if (p.accumulate) {
                float4 old = *reinterpret_cast<float4*>(o + j);
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
              }
              *reinterpret_cast<float4*>(o + j) = v;
            } else {
              for (int jj = j; jj < j + 4 && col0 + jj < p.N; ++jj)
                o[jj] = __uint_as_float(r[jj]) + (p.accumulate ? o[jj] : 0.f);
            }
          }
        } else {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + out_row * p.ldo + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j + 8 <= p.N) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j + e]);
              if (p.accumulate) {
                uint4 old = *reinterpret_cast<uint4*>(o + j);
                float2 a0 = unpack_bf16(old.x), a1 = unpack_bf16(old.y), a2 = unpack_bf16(old.z), a3 = unpack_bf16(old.w);
                f[0] += a0.x; f[1] += a0.y; f[2] += a1.x; f[3] += a1.y;
                f[4] += a2.x; f[5] += a2.y; f[6] += a3.x; f[7] += a3.y;
              }
              uint4 v = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
              *reinterpret_cast<uint4*>(o + j) = v;
            } else {
              for (int jj = j; jj < j + 8 && col0 + jj < p.N; ++jj) {
                float v = __uint_as_float(r[jj]) + (p.accumulate ? __bfloat162float(o[jj]) : 0.f);
                o[jj] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ host side
static void launch(bool a_mn, bool b_mn, int mode, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int tiles,
                   cudaStream_t stream, const CUtensorMap* ta2 = nullptr, const CUtensorMap* tb2 = nullptr) {
  const CUtensorMap& xa2 = ta2 ? *ta2 : ta;   // unused by the kernel unless p.K2 > 0
  const CUtensorMap& xb2 = tb2 ? *tb2 : tb;
  int grid = std::min(tiles, num_sms());
  if (grid <= 0) return;
#define TK_LAUNCH(AM, BMN, MD)                                                                                   \
  do {                                                                                                           \
    static bool configured = false;                                                                              \
    auto kern = gemm_tcgen05_kernel<AM, BMN, MD>;                                                                \
    if (!configured) {                                                                                           \
      TK_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));        \
      configured = true;                                                                                         \
    }                                                                                                            \
    kern<<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ta, tb, xa2, xb2, p);                                        \
  } while (0)
  if (mode == 0) {
    if (!a_mn && !b_mn) TK_LAUNCH(false, false, 0);
    else if (!a_mn && b_mn) TK_LAUNCH(false, true, 0);
    else if (a_mn && b_mn) TK_LAUNCH(true, true, 0);
    else TORCH_CHECK(false, "unsupported GEMM layout");
  } else if (mode == 1) {
    if (!a_mn && !b_mn) TK_LAUNCH(false, false, 1);
    else if (!a_mn && b_mn) TK_LAUNCH(false, true, 1);
    else TORCH_CHECK(false, "unsupported grouped GEMM layout");
  } else {
    TORCH_CHECK(a_mn && b_mn, "grouped wgrad is TN");
    TK_LAUNCH(true, true, 2);
  }
#undef TK_LAUNCH
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
}

static void check_operand(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16, name, " must be a CUDA bf16 tensor");
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with unit inner stride");
  TORCH_CHECK((t.stride(0) * 2) % 16 == 0, name, ": row pitch must be a multiple of 16 bytes (cols % 8 == 0)");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must be 16-byte aligned");
}

bool gemm_pair_launch(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, void* out, int M, int N, int K, int ldo,
                      bool out_fp32, bool accumulate, cudaStream_t stream);

// 0: single-CTA tiles only; 1: SM-pair kernel (gemm2.cu) for shapes with enough 256x256 tiles to fill the device.
static int g_pair_mode = [] {
  const char* e = getenv("TK_GEMM_PAIR");
  return e ? atoi(e) : 1;
}();
void set_gemm_pair(int64_t mode) { g_pair_mode = static_cast<int>(mode); }

// out = a·bᵀ (nt) | a·b (nn) | aᵀ·b (tn)
torch::Tensor gemm(const torch::Tensor& a, const torch::Tensor& b, const std::string& layout,
                   const c10::optional<torch::Tensor>& out_opt, bool accumulate, c10::optional<torch::ScalarType> out_dtype) {
  check_operand(a, "a");
  check_operand(b, "b");
  c10::cuda::CUDAGuard guard(a.device());
  int M, N, K;
  bool a_mn, b_mn;
  if (layout == "nt") { M = a.size(0); K = a.size(1); N = b.size(0); TORCH_CHECK(b.size(1) == K, "nt: K mismatch"); a_mn = false; b_mn = false; }
  else if (layout == "nn") { M = a.size(0); K = a.size(1); N = b.size(1); TORCH_CHECK(b.size(0) == K, "nn: K mismatch"); a_mn = false; b_mn = true; }
  else if (layout == "tn") { K = a.size(0); M = a.size(1); N = b.size(1); TORCH_CHECK(b.size(0) == K, "tn: K mismatch"); a_mn = true; b_mn = true; }
  else TORCH_CHECK(false, "layout must be nt|nn|tn");
  torch::Tensor out;
  if (out_opt.has_value()) {
    out = *out_opt;
    TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.stride(1) == 1, "bad out");
  } else {
    TORCH_CHECK(!accumulate, "accumulate needs out");
    out = torch::empty({M, N}, a.options().dtype(out_dtype.value_or(torch::kBFloat16)));
  }
  bool fp32 = out.scalar_type() == torch::kFloat32;
  TORCH_CHECK(fp32 || out.scalar_type() == torch::kBFloat16, "out must be bf16 or fp32");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0 && (out.stride(0) * out.element_size()) % 16 == 0,
              "out rows must be 16-byte aligned");
  if (M == 0 || N == 0) return out;
  if (K == 0) { if (!accumulate) out.zero_(); return out; }
  if (g_pair_mode && ((M + 255) / 256) * ((N + 255) / 256) >= num_sms() / 2) {
    CUtensorMap pa = a_mn ? make_tmap_2d(a.data_ptr(), a.size(1), a.size(0), a.stride(0), 64, BK)
                          : make_tmap_2d(a.data_ptr(), a.size(1), a.size(0), a.stride(0), BK, 128);
    CUtensorMap pb = b_mn ? make_tmap_2d(b.data_ptr(), b.size(1), b.size(0), b.stride(0), 64, BK)
                          : make_tmap_2d(b.data_ptr(), b.size(1), b.size(0), b.stride(0), BK, 128);
    if (gemm_pair_launch(a_mn, b_mn, pa, pb, out.data_ptr(), M, N, K, static_cast<int>(out.stride(0)), fp32, accumulate,
                         at::cuda::getCurrentCUDAStream()))
      return out;
  }
  // a row-major [R, C] matrix is a 2-D tensor map with dims {C, R}
  CUtensorMap ta = a_mn ? make_tmap_2d(a.data_ptr(), a.size(1), a.size(0), a.stride(0), 64, BK)
                        : make_tmap_2d(a.data_ptr(), a.size(1), a.size(0), a.stride(0), BK, BM);
  CUtensorMap tb = b_mn ? make_tmap_2d(b.data_ptr(), b.size(1), b.size(0), b.stride(0), 64, BK)
                        : make_tmap_2d(b.data_ptr(), b.size(1), b.size(0), b.stride(0), BK, BN);
  GemmParams p{};
  p.out = out.data_ptr(); p.M = M; p.N = N; p.K = K; p.ldo = out.stride(0); p.out_fp32 = fp32; p.accumulate = accumulate;
  p.err = error_word(); p.offsets = nullptr; p.num_groups = 1; p.group_rows_b = 0; p.mode = 0; p.group_map = nullptr;
  int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  launch(a_mn, b_mn, 0, ta, tb, p, tiles, at::cuda::getCurrentCUDAStream());
  return out;
}

// Expert-grouped GEMM.  x [R, K] with expert e owning rows [offsets[e], offsets[e+1]) (offsets multiples of 128;
// padding rows are zero); weight [E, N, K] (nt) or [E, K, N] (nn).  Returns [R, N].
// Optional second pair (x2 [R, K2], w2 [E, N, K2] (nt) or [E, K2, N] (nn)): returns x·W + x2·W2 from one pass — the sum
// is formed in tensor memory, the output is written once.
torch::Tensor grouped_gemm(const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& offsets, const std::string& layout,
                           const c10::optional<torch::Tensor>& group_map, const c10::optional<torch::Tensor>& out_opt, bool accumulate,
                           const c10::optional<torch::Tensor>& x2_opt, const c10::optional<torch::Tensor>& w2_opt) {
  check_operand(x, "x");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kBFloat16 && w.dim() == 3 && w.is_contiguous(), "weight [E, *, *] bf16 contiguous");
  TORCH_CHECK(offsets.is_cuda() && offsets.scalar_type() == torch::kInt32 && offsets.is_contiguous(), "offsets int32 on device");
  c10::cuda::CUDAGuard guard(x.device());
  const int R = x.size(0), K = x.size(1);
  const bool mapped = group_map.has_value() && group_map->defined();
  const int E = mapped ? static_cast<int>(group_map->numel()) : static_cast<int>(w.size(0));
  if (mapped) TORCH_CHECK(group_map->is_cuda() && group_map->scalar_type() == torch::kInt32 && group_map->is_contiguous(), "group_map int32 on device");
  TORCH_CHECK(offsets.numel() == E + 1, "offsets must have one more entry than there are groups");
  int N;
  bool b_mn;
  if (layout == "nt") { N = w.size(1); TORCH_CHECK(w.size(2) == K, "nt: K mismatch"); b_mn = false; }
  else if (layout == "nn") { N = w.size(2); TORCH_CHECK(w.size(1) == K, "nn: K mismatch"); b_mn = true; }
  else TORCH_CHECK(false, "grouped layout must be nt|nn");
  // with a map some groups may be skipped (no adapter): their rows must read as zero
  torch::Tensor out;
  if (out_opt.has_value() && out_opt->defined()) {
    out = *out_opt;  // `accumulate`: out += x·W (rows outside every group keep their value)
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kBFloat16 && out.dim() == 2 && out.size(0) == R && out.size(1) == N && out.is_contiguous(),
                "out must be [R, N] bf16 contiguous");
  } else {
    TORCH_CHECK(!accumulate, "accumulate needs out");
    out = mapped ? torch::zeros({R, N}, x.options()) : torch::empty({R, N}, x.options());
  }
  if (R == 0) return out;
  auto w2 = w.view({w.size(0) * w.size(1), w.size(2)});
  check_operand(w2, "weight");
  CUtensorMap ta = make_tmap_2d(x.data_ptr(), x.size(1), x.size(0), x.stride(0), BK, BM);
  CUtensorMap tb = b_mn ? make_tmap_2d(w2.data_ptr(), w2.size(1), w2.size(0), w2.stride(0), 64, BK)
                        : make_tmap_2d(w2.data_ptr(), w2.size(1), w2.size(0), w2.stride(0), BK, BN);
  GemmParams p{};
  p.out = out.data_ptr(); p.M = R; p.N = N; p.K = K; p.ldo = N; p.out_fp32 = 0; p.accumulate = accumulate ? 1 : 0; p.err = error_word();
  p.offsets = offsets.data_ptr<int>(); p.num_groups = E; p.group_rows_b = w.size(1); p.mode = 1;
  p.group_map = mapped ? group_map->data_ptr<int>() : nullptr;
  // upper bound of tiles: every expert wastes at most one partial M-tile
  int tiles = ((R + BM - 1) / BM + E) * ((N + BN - 1) / BN);
  const bool dual = x2_opt.has_value() && x2_opt->defined();
  if (!dual) {
    launch(false, b_mn, 1, ta, tb, p, tiles, at::cuda::getCurrentCUDAStream());
    return out;
  }
  TORCH_CHECK(w2_opt.has_value() && w2_opt->defined(), "second pair needs both operands");
  const torch::Tensor& x2 = *x2_opt;
  const torch::Tensor& wb = *w2_opt;
  check_operand(x2, "x2");
  TORCH_CHECK(x2.size(0) == R, "x2 rows");
  TORCH_CHECK(wb.is_cuda() && wb.scalar_type() == torch::kBFloat16 && wb.dim() == 3 && wb.is_contiguous() && wb.size(0) == w.size(0),
              "w2 [E, *, *] bf16 contiguous with the first pair's group count");
  const int K2 = x2.size(1);
  if (b_mn) {
    TORCH_CHECK(wb.size(1) == K2 && wb.size(2) == N, "nn: w2 must be [E, K2, N]");
  } else {
    TORCH_CHECK(wb.size(1) == N && wb.size(2) == K2, "nt: w2 must be [E, N, K2]");
  }
  auto wb2 = wb.view({wb.size(0) * wb.size(1), wb.size(2)});
  check_operand(wb2, "w2");
  CUtensorMap ta2 = make_tmap_2d(x2.data_ptr(), x2.size(1), x2.size(0), x2.stride(0), BK, BM);
  CUtensorMap tb2 = b_mn ? make_tmap_2d(wb2.data_ptr(), wb2.size(1), wb2.size(0), wb2.stride(0), 64, BK)
                         : make_tmap_2d(wb2.data_ptr(), wb2.size(1), wb2.size(0), wb2.stride(0), BK, BN);
  p.K2 = K2;
  p.group_rows_b2 = wb.size(1);
  launch(false, b_mn, 1, ta, tb, p, tiles, at::cuda::getCurrentCUDAStream(), &ta2, &tb2);
  return out;
}

// Per-expert weight gradient: dW[e] = dy[rows_e]ᵀ · x[rows_e]  → [E, N, K] fp32.  Padding rows must be zero in dy or x.
torch::Tensor grouped_gemm_wgrad(const torch::Tensor& dy, const torch::Tensor& x, const torch::Tensor& offsets, int64_t E) {
  check_operand(dy, "dy");
  check_operand(x, "x");
  TORCH_CHECK(dy.size(0) == x.size(0), "row mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  const int N = dy.size(1), K = x.size(1);
  auto out = torch::empty({E, N, K}, x.options().dtype(torch::kFloat32));
  CUtensorMap ta = make_tmap_2d(dy.data_ptr(), dy.size(1), dy.size(0), dy.stride(0), 64, BK);
  CUtensorMap tb = make_tmap_2d(x.data_ptr(), x.size(1), x.size(0), x.stride(0), 64, BK);
  GemmParams p{};
  p.out = out.data_ptr(); p.M = N; p.N = K; p.K = dy.size(0); p.ldo = K; p.out_fp32 = 1; p.accumulate = 0; p.err = error_word();
  p.offsets = offsets.data_ptr<int>(); p.num_groups = static_cast<int>(E); p.group_rows_b = 0; p.mode = 2; p.group_map = nullptr;
  int tiles = static_cast<int>(E) * ((N + BM - 1) / BM) * ((K + BN - 1) / BN);
  launch(true, true, 2, ta, tb, p, tiles, at::cuda::getCurrentCUDAStream());
  return out;
}

}  // namespace tk
