// Flash-attention forward for sm_100a: causal, GQA, packed variable-length sequences, D = 128.
//
// One CTA per (128-row query tile of one sequence, query head).  192 threads:
//   warps 0-3  softmax: thread = one query row; reads S from tensor memory (tcgen05.ld), keeps the
//              running max / sum, writes P (bf16) into a 128-byte-swizzled smem tile, rescales the O
//              accumulator in tensor memory only when a row maximum grows by more than 2^8
//   warp 4     TMA producer: Q once, then K/V tiles (double buffered)
//   warp 5     MMA issuer: S_j = Q·K_jᵀ into one of two TMEM buffers (so S_{j+1} is computed while
//              the softmax of S_j runs), O += P_j·V_j into a third TMEM buffer
// Tensor memory: S0 [0,128), S1 [128,256), O [256,384) fp32 columns.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace tk {

using bf16 = __nv_bfloat16;

namespace fa {
constexpr int BQ = 128, BKV = 128, D = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;  // 32 KiB, two [128][64] swizzle atoms
constexpr int ATOM_BYTES = 128 * 64 * 2;   // 16 KiB
constexpr int SMEM_Q = 0, SMEM_K = TILE_BYTES, SMEM_V = 3 * TILE_BYTES, SMEM_P = 5 * TILE_BYTES, SMEM_BAR = 6 * TILE_BYTES;
constexpr int SMEM_XCHG = SMEM_BAR + 256;           // row max (2 parities x 2 halves x 128) + row sums (2 x 128) floats
constexpr int SMEM_TOTAL = SMEM_XCHG + 6 * 128 * 4 + 1024;
constexpr int THREADS = 320;  // warps 0-7 softmax (two groups of 4: each owns 64 of the 128 S columns), 8 producer, 9 MMA
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units
}  // namespace fa

struct FwdParams {
  bf16* out;          // [T, Hq, D]
  float* lse;         // [Hq, T]  natural-log LSE of the scaled scores
  const int* cu;      // [n+1] query boundaries
  const int* cu_k;    // [n+1] key/value boundaries (== cu for self-attention over the same packing)
  int T, hq, hkv;
  float scale_log2;   // softmax scale · log2(e)
  int causal;
  int* err;
};

__global__ void __launch_bounds__(fa::THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using namespace fa;
  const int head = blockIdx.x, seq = blockIdx.z;
  const int seq_start = p.cu[seq], seq_len = p.cu[seq + 1] - seq_start;
  // longest-first: the heaviest (last) query tiles are scheduled first
  const int n_qtiles = (seq_len + BQ - 1) / BQ;
  if (static_cast<int>(blockIdx.y) >= n_qtiles) return;
  const int qt = n_qtiles - 1 - blockIdx.y;
  const int q0 = qt * BQ;
  const int kv_head = head / (p.hq / p.hkv);
  // keys may be longer than queries (a query chunk against a key prefix): the causal diagonal is aligned to the
  // bottom-right corner, i.e. query row r sees keys 0 … r + q_off
  const int kv_start = p.cu_k[seq], kv_len = p.cu_k[seq + 1] - kv_start;
  const int q_off = kv_len - seq_len;
  const int kv_end = p.causal ? max(0, min(kv_len, q0 + BQ + q_off)) : kv_len;
  const int n_blocks = (kv_end + BKV - 1) / BKV;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* v_full = bars + 3;        // 2
  uint64_t* kv_empty = bars + 5;      // 2
  uint64_t* s_full = bars + 7;        // 2
  uint64_t* s_empty = bars + 9;       // 2
  uint64_t* p_ready = bars + 11;      // 1
  uint64_t* o_done = bars + 12;       // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 256);
    }
    mbar_init(p_ready, 256);
    mbar_init(o_done, 1);
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 8) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_3d(smem + SMEM_Q, &tmQ, q_full, 0, head, seq_start + q0);
      tma_load_3d(smem + SMEM_Q + ATOM_BYTES, &tmQ, q_full, 64, head, seq_start + q0);
      for (int j = 0; j < n_blocks; ++j) {
        const int st = j & 1;
        if (j >= 2 && !mbar_wait(&kv_empty[st], ((j >> 1) - 1) & 1, p.err, ERR_ATTN_WAIT)) break;
        const int row = kv_start + j * BKV;
        mbar_expect_tx(&k_full[st], TILE_BYTES);
        tma_load_3d(smem + SMEM_K + st * TILE_BYTES, &tmK, &k_full[st], 0, kv_head, row);
        tma_load_3d(smem + SMEM_K + st * TILE_BYTES + ATOM_BYTES, &tmK, &k_full[st], 64, kv_head, row);
        mbar_expect_tx(&v_full[st], TILE_BYTES);
        tma_load_3d(smem + SMEM_V + st * TILE_BYTES, &tmV, &v_full[st], 0, kv_head, row);
        tma_load_3d(smem + SMEM_V + st * TILE_BYTES + ATOM_BYTES, &tmV, &v_full[st], 64, kv_head, row);
      }
    }
  } else if (warp == 9) {
    // ----------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(BQ, D, false, true);
      const uint32_t sq = smem_u32(smem + SMEM_Q), sp = smem_u32(smem + SMEM_P);
      auto issue_s = [&](int j) {
        const uint32_t sk = smem_u32(smem + SMEM_K + (j & 1) * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * ATOM_BYTES + (k & 3) * 32;
          umma_bf16(tmem_base + (j & 1) * 128, umma_desc(sq + off, 16, 1024), umma_desc(sk + off, 16, 1024), idesc_s, k ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
      };
      bool ok = mbar_wait(q_full, 0, p.err, ERR_ATTN_WAIT) && mbar_wait(&k_full[0], 0, p.err, ERR_ATTN_WAIT);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < n_blocks; ++j) {
        if (j + 1 < n_blocks) {
          const int n = j + 1;
          ok = mbar_wait(&k_full[n & 1], (n >> 1) & 1, p.err, ERR_ATTN_WAIT);
          if (ok && n >= 2) ok = mbar_wait(&s_empty[n & 1], ((n >> 1) - 1) & 1, p.err, ERR_ATTN_WAIT);
          if (!ok) break;
          tc_fence_after();
          issue_s(n);
        }
        ok = mbar_wait(p_ready, j & 1, p.err, ERR_ATTN_WAIT) && mbar_wait(&v_full[j & 1], (j >> 1) & 1, p.err, ERR_ATTN_WAIT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + SMEM_V + (j & 1) * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // A = P (K-major over kv): atom k/4, 32-byte step inside; B = V (MN-major): 16 kv rows = 2048 B per step
          const uint64_t ad = umma_desc(sp + (k >> 2) * ATOM_BYTES + (k & 3) * 32, 16, 1024);
          const uint64_t bd = umma_desc(sv + k * 2048, ATOM_BYTES, 1024);
          umma_bf16(tmem_o, ad, bd, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(o_done);
        umma_commit(&kv_empty[j & 1]);
      }
    }
  } else {
    // -------------------------------------------------------------- softmax
    // Thread = (query row, half of the 128 key columns).  The 64 scores of its half stay in registers from the
    // max pass to the exp pass (one TMEM read per block); the two halves of a row agree on the row maximum
    // through shared memory + one named barrier per block.  A thread whose wait failed keeps taking part in the
    // barriers (doing no work) so that no thread is ever left waiting at one.
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;          // row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int q_pos = q0 + row;                      // position inside the sequence
    float* xmax = reinterpret_cast<float*>(smem + SMEM_XCHG);   // [parity][half][128]
    float* xsum = xmax + 4 * 128;                                 // [half][128]
    float m_used = -INFINITY, l_sum = 0.f;
    bool dead = false;
    for (int j = 0; j < n_blocks; ++j) {
      if (!dead && !mbar_wait(&s_full[j & 1], (j >> 1) & 1, p.err, ERR_ATTN_WAIT)) dead = true;
      const int kv0 = j * BKV + wg * 64;
      float sc[64];
      float mx = -INFINITY;
      if (!dead) {
        tc_fence_after();
        const uint32_t ts = tmem_base + (j & 1) * 128 + wg * 64 + lane_off;
        uint32_t r0[32], r1[32];
        tmem_ld32(ts, r0);
        tmem_ld32(ts + 32, r1);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&s_empty[j & 1]);                 // scores are in registers: the TMEM buffer may be refilled
        const bool need_mask = (kv0 + 64 > kv_end) || (p.causal && kv0 + 64 > q0 + q_off);
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float sv = __uint_as_float(i < 32 ? r0[i] : r1[i - 32]) * p.scale_log2;
          if (need_mask) {
            const int col = kv0 + i;
            if (col >= kv_end || (p.causal && col > q_pos + q_off)) sv = -INFINITY;
          }
          sc[i] = sv;
          mx = fmaxf(mx, sv);
        }
      }
      xmax[((j & 1) * 2 + wg) * 128 + row] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(mx, xmax[((j & 1) * 2 + (wg ^ 1)) * 128 + row]);
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + RESCALE_THRESHOLD || m_used == -INFINITY) {
        const float m_new = (mx == -INFINITY) ? 0.f : mx;   // fully masked (garbage) rows stay finite
        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
        rescale = (j > 0);
        m_used = m_new;
        l_sum *= alpha;
      }
      // P buffer and O accumulator are free once the previous P·V has retired
      if (!dead && j > 0 && !mbar_wait(o_done, (j - 1) & 1, p.err, ERR_ATTN_WAIT)) dead = true;
      if (dead) continue;
      tc_fence_after();
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_o + lane_off + wg * 64 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tmem_o + lane_off + wg * 64 + c * 32, r);
        }
        tmem_st_wait();
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fast_exp2(sc[c * 32 + i] - m_used), p1 = fast_exp2(sc[c * 32 + i + 1] - m_used);
          // the sum uses the bf16-rounded values so that numerator and denominator match
          const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          l_sum += __low2float(pb) + __high2float(pb);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        store_row_chunk_sw128(smem + SMEM_P, 128, row, wg * 64 + c * 32, packed);
      }
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(p_ready);
    }
    // ------------------------------------------------------------- epilogue
    xsum[wg * 128 + row] = l_sum;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l_sum += xsum[(wg ^ 1) * 128 + row];
    if (!dead && n_blocks > 0 && mbar_wait(o_done, (n_blocks - 1) & 1, p.err, ERR_ATTN_WAIT)) {
      tc_fence_after();
      const float inv_l = (l_sum > 0.f) ? 1.f / l_sum : 0.f;
      const bool valid = q_pos < seq_len;
      bf16* orow = p.out + (static_cast<size_t>(seq_start + q_pos) * p.hq + head) * D;
#pragma unroll 1
      for (int c = 2 * wg; c < 2 * wg + 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_o + lane_off + c * 32, r);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v = make_uint4(pack_bf16(__uint_as_float(r[i]) * inv_l, __uint_as_float(r[i + 1]) * inv_l),
                                 pack_bf16(__uint_as_float(r[i + 2]) * inv_l, __uint_as_float(r[i + 3]) * inv_l),
                                 pack_bf16(__uint_as_float(r[i + 4]) * inv_l, __uint_as_float(r[i + 5]) * inv_l),
                                 pack_bf16(__uint_as_float(r[i + 6]) * inv_l, __uint_as_float(r[i + 7]) * inv_l));
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = v;
          }
        }
      }
      if (valid && wg == 0) p.lse[static_cast<size_t>(head) * p.T + seq_start + q_pos] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dims {D, H, T}: a box {64, 1, 128} is a [128 tokens][64] K-major swizzle atom of one head.
CUtensorMap make_head_tmap(const torch::Tensor& t, int rows) {
  return make_tmap_3d(t.data_ptr(), t.size(2), t.size(1), t.size(0), t.stride(1), t.stride(0), 64, 1, rows);
}

std::vector<torch::Tensor> flash_attn_fwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, const torch::Tensor& cu,
                                          int64_t max_seqlen, bool causal, double scale, const c10::optional<torch::Tensor>& cu_k) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == torch::kBFloat16 && q.dim() == 3 && q.is_contiguous(), "q [T,Hq,128] bf16 contiguous");
  TORCH_CHECK(k.is_contiguous() && v.is_contiguous() && k.sizes() == v.sizes() && k.scalar_type() == torch::kBFloat16, "k/v [T,Hkv,128]");
  TORCH_CHECK(q.size(2) == 128 && k.size(2) == 128, "head_dim must be 128");
  TORCH_CHECK(cu.is_cuda() && cu.scalar_type() == torch::kInt32 && cu.is_contiguous(), "cu_seqlens int32 on device");
  TORCH_CHECK(q.size(1) % k.size(1) == 0, "Hq must be a multiple of Hkv");
  c10::cuda::CUDAGuard guard(q.device());
  const int T = q.size(0), hq = q.size(1), hkv = k.size(1), nseq = cu.numel() - 1;
  auto out = torch::empty_like(q);
  auto lse = torch::empty({hq, T}, q.options().dtype(torch::kFloat32));
  if (T == 0 || nseq <= 0) return {out, lse};
  CUtensorMap tq = make_head_tmap(q, 128), tk_ = make_head_tmap(k, 128), tv = make_head_tmap(v, 128);
  FwdParams p{};
  p.out = reinterpret_cast<bf16*>(out.data_ptr()); p.lse = lse.data_ptr<float>(); p.cu = cu.data_ptr<int>();
  p.cu_k = p.cu;
  if (cu_k.has_value() && cu_k->defined()) {
    TORCH_CHECK(cu_k->is_cuda() && cu_k->scalar_type() == torch::kInt32 && cu_k->is_contiguous() && cu_k->numel() == cu.numel(), "cu_k like cu");
    p.cu_k = cu_k->data_ptr<int>();
  }
  p.T = T; p.hq = hq; p.hkv = hkv; p.scale_log2 = static_cast<float>(scale * 1.4426950408889634); p.causal = causal; p.err = error_word();
  static bool configured = false;
  if (!configured) {
    TK_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::SMEM_TOTAL));
    configured = true;
  }
  dim3 grid(hq, (static_cast<int>(max_seqlen) + fa::BQ - 1) / fa::BQ, nseq);
  flash_fwd_kernel<<<grid, fa::THREADS, fa::SMEM_TOTAL, at::cuda::getCurrentCUDAStream()>>>(tq, tk_, tv, p);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return {out, lse};
}

}  // namespace tk
