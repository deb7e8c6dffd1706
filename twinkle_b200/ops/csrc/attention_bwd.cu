// Flash-attention backward for sm_100a (causal, GQA, packed varlen, D = 128), two tcgen05 kernels:
//
//   flash_bwd_dkdv_kernel : one CTA per (128-row K/V tile, kv head).  Loops over the query heads of the
//       GQA group and over 64-row query blocks:  Sᵀ = K·Qᵀ, dPᵀ = V·dOᵀ (tensor cores → TMEM),
//       Pᵀ = exp2(Sᵀ·c − lse), dSᵀ = Pᵀ∘(dPᵀ − δ) (registers → swizzled smem), dV += Pᵀ·dO, dK += dSᵀ·Q.
//       dK/dV of the whole group accumulate in TMEM → no atomics, deterministic.
//   flash_bwd_dq_kernel   : one CTA per (128-row query tile, query head).  Loops over 64-row K/V blocks:
//       S = Q·Kᵀ, dP = dO·Vᵀ, dS = P∘(dP − δ), dQ += dS·K.
//   flash_bwd_delta_kernel: δ[h,t] = Σ_d O·dO.
// Recomputing S/dP in both kernels costs 7 instead of 5 GEMMs per tile pair but keeps every
// accumulator on chip without cross-CTA reductions.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace tk {

using bf16 = __nv_bfloat16;
CUtensorMap make_head_tmap(const torch::Tensor& t, int rows);

namespace fb {
constexpr int D = 128, BT = 128 /*outer tile rows*/, BI = 64 /*inner block rows*/;
constexpr int OUTER_BYTES = BT * D * 2;       // 32 KiB (two [128][64] atoms)
constexpr int OUTER_ATOM = BT * 64 * 2;       // 16 KiB
constexpr int INNER_BYTES = BI * D * 2;       // 16 KiB (two [64][64] atoms)
constexpr int INNER_ATOM = BI * 64 * 2;       // 8 KiB
constexpr int PT_BYTES = BT * BI * 2;         // 16 KiB ([128][64] atom)
constexpr int THREADS = 320;  // warps 0-7 compute (two groups of 4, each takes half of the inner-block columns), 8 producer, 9 MMA
// dkdv: K, V (outer) | Q×2, dO×2 (inner) | Pᵀ, dSᵀ | lse/delta staging | barriers
constexpr int KV_SMEM_K = 0, KV_SMEM_V = OUTER_BYTES, KV_SMEM_Q = 2 * OUTER_BYTES, KV_SMEM_DO = KV_SMEM_Q + 2 * INNER_BYTES,
              KV_SMEM_PT = KV_SMEM_DO + 2 * INNER_BYTES, KV_SMEM_DST = KV_SMEM_PT + PT_BYTES, KV_SMEM_STAT = KV_SMEM_DST + PT_BYTES,
              KV_SMEM_BAR = KV_SMEM_STAT + 2 * 2 * BI * 4, KV_SMEM_TOTAL = KV_SMEM_BAR + 256 + 1024;
// dq: Q, dO (outer) | K×2, V×2 (inner) | dS | barriers
constexpr int DQ_SMEM_Q = 0, DQ_SMEM_DO = OUTER_BYTES, DQ_SMEM_K = 2 * OUTER_BYTES, DQ_SMEM_V = DQ_SMEM_K + 2 * INNER_BYTES,
              DQ_SMEM_DS = DQ_SMEM_V + 2 * INNER_BYTES, DQ_SMEM_BAR = DQ_SMEM_DS + PT_BYTES, DQ_SMEM_TOTAL = DQ_SMEM_BAR + 256 + 1024;
}  // namespace fb

struct BwdParams {
  bf16 *dq, *dk, *dv;    // [T,Hq,D], [T,Hkv,D], [T,Hkv,D]
  const float* lse;      // [Hq,T] natural log
  const float* delta;    // [Hq,T]
  const int* cu;
  int T, hq, hkv;
  float scale, scale_log2;
  int causal;
  const int* cu_k;   // key/value boundaries (== cu for self-attention over the same packing)
  int* err;
};

__global__ void flash_bwd_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout, float* __restrict__ delta, int T, int hq) {
  // one warp per (token, head); 128 elements → 4 per lane
  const long total = static_cast<long>(T) * hq;
  const int lane = threadIdx.x & 31;
  for (long item = static_cast<long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); item < total;
       item += static_cast<long>(gridDim.x) * (blockDim.x >> 5)) {
    const uint2 a = *reinterpret_cast<const uint2*>(o + item * 128 + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(dout + item * 128 + lane * 4);
    float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y);
    float s = warp_sum(a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y);
    if (lane == 0) {
      const int t = static_cast<int>(item / hq), h = static_cast<int>(item % hq);
      delta[static_cast<size_t>(h) * T + t] = s;
    }
  }
}

// ============================================================== dK / dV
__global__ void __launch_bounds__(fb::THREADS, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
  using namespace fb;
  const int kv_head = blockIdx.x, seq = blockIdx.z;
  const int seq_start = p.cu[seq], seq_len = p.cu[seq + 1] - seq_start;          // queries
  const int kv_start = p.cu_k[seq], kv_len = p.cu_k[seq + 1] - kv_start;         // keys / values
  const int q_off = kv_len - seq_len;            // causal: query row r sees keys 0 … r + q_off
  const int n_tiles = (kv_len + BT - 1) / BT;
  if (static_cast<int>(blockIdx.y) >= n_tiles) return;
  const int kv0 = blockIdx.y * BT;               // early tiles have the most query blocks → scheduled first
  const int G = p.hq / p.hkv;
  const int qb_end = (seq_len + BI - 1) / BI;
  const int qb_begin = p.causal ? min(max(kv0 - q_off, 0) / BI, qb_end) : 0;
  const int per_head = qb_end - qb_begin;
  const int n_iter = per_head * G;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + KV_SMEM_BAR);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // 2
  uint64_t* qdo_empty = bars + 3;    // 2
  uint64_t* sd_full = bars + 5;      // 2
  uint64_t* sd_empty = bars + 7;     // 2
  uint64_t* pds_ready = bars + 9;    // 1
  uint64_t* acc_done = bars + 10;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  float* stat = reinterpret_cast<float*>(smem + KV_SMEM_STAT);  // [2 buffers][lse2 | delta][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&sd_full[i], 1);
      mbar_init(&sd_empty[i], 256);
    }
    mbar_init(pds_ready, 256);
    mbar_init(acc_done, 1);
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
  // TMEM columns: Sᵀ buffers [0,64) [64,128); dPᵀ buffers [128,192) [192,256); dV [256,384); dK [384,512)
  const uint32_t t_dv = tmem_base + 256, t_dk = tmem_base + 384;

  if (warp == 8) {
    // producer warp: lane 0 drives TMA; all lanes stage lse (log2 units) and δ of each query block in smem
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * OUTER_BYTES);
      tma_load_3d(smem + KV_SMEM_K, &tmK, kv_full, 0, kv_head, kv_start + kv0);
      tma_load_3d(smem + KV_SMEM_K + OUTER_ATOM, &tmK, kv_full, 64, kv_head, kv_start + kv0);
      tma_load_3d(smem + KV_SMEM_V, &tmV, kv_full, 0, kv_head, kv_start + kv0);
      tma_load_3d(smem + KV_SMEM_V + OUTER_ATOM, &tmV, kv_full, 64, kv_head, kv_start + kv0);
    }
    for (int it = 0; it < n_iter; ++it) {
      const int st = it & 1;
      if (it >= 2) {
        int ok = 1;
        if (lane == 0) ok = mbar_wait(&qdo_empty[st], ((it >> 1) - 1) & 1, p.err, ERR_ATTN_WAIT) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      const int head = kv_head * G + it / per_head;
      const int qb0 = (qb_begin + it % per_head) * BI;
      for (int c = lane; c < BI; c += 32) {
        const int qpos = qb0 + c;
        float l2 = INFINITY, dl = 0.f;   // exp2(s − inf) = 0 for query rows past the end of the sequence
        if (qpos < seq_len) {
          const size_t idx = static_cast<size_t>(head) * p.T + seq_start + qpos;
          l2 = p.lse[idx] * 1.4426950408889634f;
          dl = p.delta[idx];
        }
        stat[st * 2 * BI + c] = l2;
        stat[st * 2 * BI + BI + c] = dl;
      }
      __syncwarp();
      if (lane == 0) {
        const int row = seq_start + qb0;
        mbar_expect_tx(&qdo_full[st], 2 * INNER_BYTES);
        tma_load_3d(smem + KV_SMEM_Q + st * INNER_BYTES, &tmQ, &qdo_full[st], 0, head, row);
        tma_load_3d(smem + KV_SMEM_Q + st * INNER_BYTES + INNER_ATOM, &tmQ, &qdo_full[st], 64, head, row);
        tma_load_3d(smem + KV_SMEM_DO + st * INNER_BYTES, &tmDO, &qdo_full[st], 0, head, row);
        tma_load_3d(smem + KV_SMEM_DO + st * INNER_BYTES + INNER_ATOM, &tmDO, &qdo_full[st], 64, head, row);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BT, BI, false, false);   // [128 kv] x [64 q], K = d
      constexpr uint32_t idesc_acc = umma_idesc_bf16(BT, D, false, true);   // [128 kv] x [128 d], K = q (B MN-major)
      const uint32_t sk = smem_u32(smem + KV_SMEM_K), sv = smem_u32(smem + KV_SMEM_V);
      const uint32_t spt = smem_u32(smem + KV_SMEM_PT), sdst = smem_u32(smem + KV_SMEM_DST);
      auto issue_sd = [&](int it) {
        const int st = it & 1;
        const uint32_t sq = smem_u32(smem + KV_SMEM_Q + st * INNER_BYTES), sdo = smem_u32(smem + KV_SMEM_DO + st * INNER_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t offA = (k >> 2) * OUTER_ATOM + (k & 3) * 32, offB = (k >> 2) * INNER_ATOM + (k & 3) * 32;
          umma_bf16(tmem_base + st * 64, umma_desc(sk + offA, 16, 1024), umma_desc(sq + offB, 16, 1024), idesc_s, k ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t offA = (k >> 2) * OUTER_ATOM + (k & 3) * 32, offB = (k >> 2) * INNER_ATOM + (k & 3) * 32;
          umma_bf16(tmem_base + 128 + st * 64, umma_desc(sv + offA, 16, 1024), umma_desc(sdo + offB, 16, 1024), idesc_s, k ? 1u : 0u);
        }
        umma_commit(&sd_full[st]);
      };
      bool ok = n_iter > 0 && mbar_wait(kv_full, 0, p.err, ERR_ATTN_WAIT) && mbar_wait(&qdo_full[0], 0, p.err, ERR_ATTN_WAIT);
      if (ok) {
        tc_fence_after();
        issue_sd(0);
      }
      for (int it = 0; ok && it < n_iter; ++it) {
        if (it + 1 < n_iter) {
          const int n = it + 1;
          ok = mbar_wait(&qdo_full[n & 1], (n >> 1) & 1, p.err, ERR_ATTN_WAIT);
          if (ok && n >= 2) ok = mbar_wait(&sd_empty[n & 1], ((n >> 1) - 1) & 1, p.err, ERR_ATTN_WAIT);
          if (!ok) break;
          tc_fence_after();
          issue_sd(n);
        }
        if (!mbar_wait(pds_ready, it & 1, p.err, ERR_ATTN_WAIT)) break;
        tc_fence_after();
        const int st = it & 1;
        const uint32_t sq = smem_u32(smem + KV_SMEM_Q + st * INNER_BYTES), sdo = smem_u32(smem + KV_SMEM_DO + st * INNER_BYTES);
#pragma unroll
        for (int k = 0; k < BI / 16; ++k)   // dV += Pᵀ·dO
          umma_bf16(t_dv, umma_desc(spt + k * 32, 16, 1024), umma_desc(sdo + k * 2048, INNER_ATOM, 1024), idesc_acc, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < BI / 16; ++k)   // dK += dSᵀ·Q
          umma_bf16(t_dk, umma_desc(sdst + k * 32, 16, 1024), umma_desc(sq + k * 2048, INNER_ATOM, 1024), idesc_acc, (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(acc_done);
        umma_commit(&qdo_empty[st]);
      }
    }
  } else {
    const int wg = warp >> 2;                       // which half of the 64 inner-block columns this thread handles
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int kv_pos = kv0 + row;
    const bool row_valid = kv_pos < kv_len;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int st = it & 1;
      const int qb0 = (qb_begin + it % per_head) * BI;
      if (!mbar_wait(&sd_full[st], (it >> 1) & 1, p.err, ERR_ATTN_WAIT)) { ok = false; break; }
      tc_fence_after();
      const float* lse2 = stat + st * 2 * BI;
      const float* dl = lse2 + BI;
      {
        const int c = wg;
        uint32_t s[32], dp[32];
        tmem_ld32(tmem_base + st * 64 + c * 32 + lane_off, s);
        tmem_ld32(tmem_base + 128 + st * 64 + c * 32 + lane_off, dp);
        tmem_ld_wait();
        uint32_t pk[16], dsk[16];
        // only blocks that touch the causal diagonal need per-element masking; rows past the end of the keys are
        // zeroed wholesale; query rows past the end carry lse = +inf and vanish through exp2
        const bool diag = p.causal && (qb0 + q_off < kv0 + BT - 1);
        const float4* l4 = reinterpret_cast<const float4*>(lse2 + c * 32);
        const float4* d4 = reinterpret_cast<const float4*>(dl + c * 32);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 lv = l4[i >> 2], dv4 = d4[i >> 2];
          const float ls[4] = {lv.x, lv.y, lv.z, lv.w}, ds[4] = {dv4.x, dv4.y, dv4.z, dv4.w};
          float pv[4], dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pr = fast_exp2(__uint_as_float(s[i + e]) * p.scale_log2 - ls[e]);
            if (diag && (qb0 + c * 32 + i + e + q_off < kv_pos)) pr = 0.f;
            pv[e] = pr;
            dv[e] = pr * (__uint_as_float(dp[i + e]) - ds[e]);
          }
          pk[i >> 1] = pack_bf16(pv[0], pv[1]);
          pk[(i >> 1) + 1] = pack_bf16(pv[2], pv[3]);
          dsk[i >> 1] = pack_bf16(dv[0], dv[1]);
          dsk[(i >> 1) + 1] = pack_bf16(dv[2], dv[3]);
        }
        if (!row_valid) {
#pragma unroll
          for (int i = 0; i < 16; ++i) { pk[i] = 0u; dsk[i] = 0u; }
        }
        // S/dP are in registers: the TMEM buffers can be refilled while we finish
        tc_fence_before();
        mbar_arrive(&sd_empty[st]);
        // Pᵀ / dSᵀ smem is free once the accumulating MMAs of the previous iteration retired
        if (it > 0 && !mbar_wait(acc_done, (it - 1) & 1, p.err, ERR_ATTN_WAIT)) { ok = false; break; }
        store_row_chunk_sw128(smem + KV_SMEM_PT, 128, row, c * 32, pk);
        store_row_chunk_sw128(smem + KV_SMEM_DST, 128, row, c * 32, dsk);
      }
      fence_proxy_async();
      mbar_arrive(pds_ready);
    }
    if (ok && n_iter > 0 && mbar_wait(acc_done, (n_iter - 1) & 1, p.err, ERR_ATTN_WAIT)) {
      tc_fence_after();
      bf16* dkrow = p.dk + (static_cast<size_t>(kv_start + kv_pos) * p.hkv + kv_head) * D;
      bf16* dvrow = p.dv + (static_cast<size_t>(kv_start + kv_pos) * p.hkv + kv_head) * D;
#pragma unroll 1
      for (int c = 2 * wg; c < 2 * wg + 2; ++c) {
        uint32_t a[32], b[32];
        tmem_ld32(t_dv + lane_off + c * 32, a);
        tmem_ld32(t_dk + lane_off + c * 32, b);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            *reinterpret_cast<uint4*>(dvrow + c * 32 + i) =
                make_uint4(pack_bf16(__uint_as_float(a[i]), __uint_as_float(a[i + 1])), pack_bf16(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3])),
                           pack_bf16(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5])), pack_bf16(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7])));
            *reinterpret_cast<uint4*>(dkrow + c * 32 + i) =
                make_uint4(pack_bf16(__uint_as_float(b[i]) * p.scale, __uint_as_float(b[i + 1]) * p.scale),
                           pack_bf16(__uint_as_float(b[i + 2]) * p.scale, __uint_as_float(b[i + 3]) * p.scale),
                           pack_bf16(__uint_as_float(b[i + 4]) * p.scale, __uint_as_float(b[i + 5]) * p.scale),
                           pack_bf16(__uint_as_float(b[i + 6]) * p.scale, __uint_as_float(b[i + 7]) * p.scale));
          }
        }
      }
    } else if (n_iter == 0 && row_valid) {
      // no query attends to this tile (cannot happen with causal self-attention, kept for safety)
      bf16* dkrow = p.dk + (static_cast<size_t>(kv_start + kv_pos) * p.hkv + kv_head) * D;
      bf16* dvrow = p.dv + (static_cast<size_t>(kv_start + kv_pos) * p.hkv + kv_head) * D;
      for (int i = wg * 64; i < wg * 64 + 64; i += 8) {
        *reinterpret_cast<uint4*>(dkrow + i) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dvrow + i) = make_uint4(0, 0, 0, 0);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ==================================================================== dQ
__global__ void __launch_bounds__(fb::THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
  using namespace fb;
  const int head = blockIdx.x, seq = blockIdx.z;
  const int seq_start = p.cu[seq], seq_len = p.cu[seq + 1] - seq_start;
  const int n_tiles = (seq_len + BT - 1) / BT;
  if (static_cast<int>(blockIdx.y) >= n_tiles) return;
  const int q0 = (n_tiles - 1 - blockIdx.y) * BT;
  const int kv_head = head / (p.hq / p.hkv);
  const int kv_start = p.cu_k[seq], kv_len = p.cu_k[seq + 1] - kv_start;
  const int q_off = kv_len - seq_len;
  const int kv_end = p.causal ? max(0, min(kv_len, q0 + BT + q_off)) : kv_len;
  const int n_iter = (kv_end + BI - 1) / BI;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DQ_SMEM_BAR);
  uint64_t* qdo_full = bars;         // 1
  uint64_t* kv_full = bars + 1;      // 2
  uint64_t* kv_empty = bars + 3;     // 2
  uint64_t* sd_full = bars + 5;      // 2
  uint64_t* sd_empty = bars + 7;     // 2
  uint64_t* ds_ready = bars + 9;     // 1
  uint64_t* acc_done = bars + 10;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&sd_full[i], 1);
      mbar_init(&sd_empty[i], 256);
    }
    mbar_init(ds_ready, 256);
    mbar_init(acc_done, 1);
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
  // TMEM columns: S buffers [0,64) [64,128); dP buffers [128,192) [192,256); dQ [256,384)
  const uint32_t t_dq = tmem_base + 256;

  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(qdo_full, 2 * OUTER_BYTES);
      tma_load_3d(smem + DQ_SMEM_Q, &tmQ, qdo_full, 0, head, seq_start + q0);
      tma_load_3d(smem + DQ_SMEM_Q + OUTER_ATOM, &tmQ, qdo_full, 64, head, seq_start + q0);
      tma_load_3d(smem + DQ_SMEM_DO, &tmDO, qdo_full, 0, head, seq_start + q0);
      tma_load_3d(smem + DQ_SMEM_DO + OUTER_ATOM, &tmDO, qdo_full, 64, head, seq_start + q0);
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        if (it >= 2 && !mbar_wait(&kv_empty[st], ((it >> 1) - 1) & 1, p.err, ERR_ATTN_WAIT)) break;
        const int row = kv_start + it * BI;
        mbar_expect_tx(&kv_full[st], 2 * INNER_BYTES);
        tma_load_3d(smem + DQ_SMEM_K + st * INNER_BYTES, &tmK, &kv_full[st], 0, kv_head, row);
        tma_load_3d(smem + DQ_SMEM_K + st * INNER_BYTES + INNER_ATOM, &tmK, &kv_full[st], 64, kv_head, row);
        tma_load_3d(smem + DQ_SMEM_V + st * INNER_BYTES, &tmV, &kv_full[st], 0, kv_head, row);
        tma_load_3d(smem + DQ_SMEM_V + st * INNER_BYTES + INNER_ATOM, &tmV, &kv_full[st], 64, kv_head, row);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BT, BI, false, false);   // [128 q] x [64 kv], K = d
      constexpr uint32_t idesc_acc = umma_idesc_bf16(BT, D, false, true);   // [128 q] x [128 d], K = kv (B MN-major)
      const uint32_t sq = smem_u32(smem + DQ_SMEM_Q), sdo = smem_u32(smem + DQ_SMEM_DO), sds = smem_u32(smem + DQ_SMEM_DS);
      auto issue_sd = [&](int it) {
        const int st = it & 1;
        const uint32_t sk = smem_u32(smem + DQ_SMEM_K + st * INNER_BYTES), sv = smem_u32(smem + DQ_SMEM_V + st * INNER_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t offA = (k >> 2) * OUTER_ATOM + (k & 3) * 32, offB = (k >> 2) * INNER_ATOM + (k & 3) * 32;
          umma_bf16(tmem_base + st * 64, umma_desc(sq + offA, 16, 1024), umma_desc(sk + offB, 16, 1024), idesc_s, k ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t offA = (k >> 2) * OUTER_ATOM + (k & 3) * 32, offB = (k >> 2) * INNER_ATOM + (k & 3) * 32;
          umma_bf16(tmem_base + 128 + st * 64, umma_desc(sdo + offA, 16, 1024), umma_desc(sv + offB, 16, 1024), idesc_s, k ? 1u : 0u);
        }
        umma_commit(&sd_full[st]);
      };
      bool ok = n_iter > 0 && mbar_wait(qdo_full, 0, p.err, ERR_ATTN_WAIT) && mbar_wait(&kv_full[0], 0, p.err, ERR_ATTN_WAIT);
      if (ok) {
        tc_fence_after();
        issue_sd(0);
      }
      for (int it = 0; ok && it < n_iter; ++it) {
        if (it + 1 < n_iter) {
          const int n = it + 1;
          ok = mbar_wait(&kv_full[n & 1], (n >> 1) & 1, p.err, ERR_ATTN_WAIT);
          if (ok && n >= 2) ok = mbar_wait(&sd_empty[n & 1], ((n >> 1) - 1) & 1, p.err, ERR_ATTN_WAIT);
          if (!ok) break;
          tc_fence_after();
          issue_sd(n);
        }
        if (!mbar_wait(ds_ready, it & 1, p.err, ERR_ATTN_WAIT)) break;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + DQ_SMEM_K + (it & 1) * INNER_BYTES);
#pragma unroll
        for (int k = 0; k < BI / 16; ++k)   // dQ += dS·K
          umma_bf16(t_dq, umma_desc(sds + k * 32, 16, 1024), umma_desc(sk + k * 2048, INNER_ATOM, 1024), idesc_acc, (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(acc_done);
        umma_commit(&kv_empty[it & 1]);
      }
    }
  } else {
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int q_pos = q0 + row;
    const bool row_valid = q_pos < seq_len;
    float lse2 = INFINITY, dl = 0.f;
    if (row_valid) {
      const size_t idx = static_cast<size_t>(head) * p.T + seq_start + q_pos;
      lse2 = p.lse[idx] * 1.4426950408889634f;
      dl = p.delta[idx];
    }
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int st = it & 1;
      if (!mbar_wait(&sd_full[st], (it >> 1) & 1, p.err, ERR_ATTN_WAIT)) { ok = false; break; }
      tc_fence_after();
      const int kvb = it * BI;
      {
        const int c = wg;
        uint32_t s[32], dp[32];
        tmem_ld32(tmem_base + st * 64 + c * 32 + lane_off, s);
        tmem_ld32(tmem_base + 128 + st * 64 + c * 32 + lane_off, dp);
        tmem_ld_wait();
        uint32_t dsk[16];
        // masking is needed only where the block crosses the causal diagonal of this query tile or the end of the keys
        const bool edge = (kvb + BI > kv_len) || (p.causal && kvb + BI - 1 > q0 + q_off);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float pr = fast_exp2(__uint_as_float(s[i + e]) * p.scale_log2 - lse2);
            if (edge) {
              const int kv_pos = kvb + c * 32 + i + e;
              if (kv_pos >= kv_len || (p.causal && kv_pos > q_pos + q_off)) pr = 0.f;
            }
            dv[e] = pr * (__uint_as_float(dp[i + e]) - dl);
          }
          dsk[i >> 1] = pack_bf16(dv[0], dv[1]);
        }
        tc_fence_before();
        mbar_arrive(&sd_empty[st]);
        if (it > 0 && !mbar_wait(acc_done, (it - 1) & 1, p.err, ERR_ATTN_WAIT)) { ok = false; break; }
        store_row_chunk_sw128(smem + DQ_SMEM_DS, 128, row, c * 32, dsk);
      }
      fence_proxy_async();
      mbar_arrive(ds_ready);
    }
    if (ok && n_iter > 0 && mbar_wait(acc_done, (n_iter - 1) & 1, p.err, ERR_ATTN_WAIT)) {
      tc_fence_after();
      bf16* dqrow = p.dq + (static_cast<size_t>(seq_start + q_pos) * p.hq + head) * D;
#pragma unroll 1
      for (int c = 2 * wg; c < 2 * wg + 2; ++c) {
        uint32_t a[32];
        tmem_ld32(t_dq + lane_off + c * 32, a);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(dqrow + c * 32 + i) =
                make_uint4(pack_bf16(__uint_as_float(a[i]) * p.scale, __uint_as_float(a[i + 1]) * p.scale),
                           pack_bf16(__uint_as_float(a[i + 2]) * p.scale, __uint_as_float(a[i + 3]) * p.scale),
                           pack_bf16(__uint_as_float(a[i + 4]) * p.scale, __uint_as_float(a[i + 5]) * p.scale),
                           pack_bf16(__uint_as_float(a[i + 6]) * p.scale, __uint_as_float(a[i + 7]) * p.scale));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

std::vector<torch::Tensor> flash_attn_bwd(const torch::Tensor& dout, const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                                          const torch::Tensor& out, const torch::Tensor& lse, const torch::Tensor& cu, int64_t max_seqlen,
                                          bool causal, double scale, const c10::optional<torch::Tensor>& cu_k, int64_t max_seqlen_k) {
  TORCH_CHECK(dout.is_contiguous() && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && out.is_contiguous(), "contiguous inputs");
  TORCH_CHECK(dout.scalar_type() == torch::kBFloat16 && dout.sizes() == q.sizes(), "dout like q");
  c10::cuda::CUDAGuard guard(q.device());
  const int T = q.size(0), hq = q.size(1), hkv = k.size(1), nseq = cu.numel() - 1;
  auto dq = torch::empty_like(q), dk = torch::empty_like(k), dv = torch::empty_like(v);
  if (T == 0 || nseq <= 0) return {dq, dk, dv};
  auto stream = at::cuda::getCurrentCUDAStream();
  auto delta = torch::empty({hq, T}, q.options().dtype(torch::kFloat32));
  {
    long items = static_cast<long>(T) * hq;
    int blocks = static_cast<int>(std::min<long>((items + 7) / 8, num_sms() * 16L));
    flash_bwd_delta_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(out.data_ptr()), reinterpret_cast<const bf16*>(dout.data_ptr()),
                                                       delta.data_ptr<float>(), T, hq);
  }
  BwdParams p{};
  p.dq = reinterpret_cast<bf16*>(dq.data_ptr()); p.dk = reinterpret_cast<bf16*>(dk.data_ptr()); p.dv = reinterpret_cast<bf16*>(dv.data_ptr());
  p.lse = lse.data_ptr<float>(); p.delta = delta.data_ptr<float>(); p.cu = cu.data_ptr<int>();
  p.T = T; p.hq = hq; p.hkv = hkv; p.scale = static_cast<float>(scale); p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.causal = causal; p.err = error_word();
  p.cu_k = p.cu;
  if (cu_k.has_value() && cu_k->defined()) {
    TORCH_CHECK(cu_k->is_cuda() && cu_k->scalar_type() == torch::kInt32 && cu_k->is_contiguous() && cu_k->numel() == cu.numel(), "cu_k like cu");
    p.cu_k = cu_k->data_ptr<int>();
  }
  static bool configured = false;
  if (!configured) {
    TK_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fb::KV_SMEM_TOTAL));
    TK_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fb::DQ_SMEM_TOTAL));
    configured = true;
  }
  const int tiles = (static_cast<int>(max_seqlen) + fb::BT - 1) / fb::BT;
  const int tiles_k = (static_cast<int>(max_seqlen_k > 0 ? max_seqlen_k : max_seqlen) + fb::BT - 1) / fb::BT;
  {
    CUtensorMap tq = make_head_tmap(q, fb::BI), tdo = make_head_tmap(dout, fb::BI), tk_ = make_head_tmap(k, fb::BT), tv = make_head_tmap(v, fb::BT);
    dim3 grid(hkv, tiles_k, nseq);
    flash_bwd_dkdv_kernel<<<grid, fb::THREADS, fb::KV_SMEM_TOTAL, stream>>>(tq, tk_, tv, tdo, p);
  }
  {
    CUtensorMap tq = make_head_tmap(q, fb::BT), tdo = make_head_tmap(dout, fb::BT), tk_ = make_head_tmap(k, fb::BI), tv = make_head_tmap(v, fb::BI);
    dim3 grid(hq, tiles, nseq);
    flash_bwd_dq_kernel<<<grid, fb::THREADS, fb::DQ_SMEM_TOTAL, stream>>>(tq, tk_, tv, tdo, p);
  }
  count_launch(3);
  TK_CUDA_CHECK(cudaGetLastError());
  return {dq, dk, dv};
}

}  // namespace tk
