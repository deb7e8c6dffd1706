// bf16 GEMM with SM pairs: tcgen05.mma.cta_group::2 on 256x256 output tiles (dense mode of gemm.cu's kernel).
//
// A thread-block cluster of two CTAs (one SM each) owns one 256x256 tile of D.  CTA r of the pair loads rows
// [128r, 128r+128) of the A tile and rows [128r, 128r+128) of the B tile, so one SM pulls 32 KB of operands per
// 256x256x64 step instead of the 48 KB a 128x256 single-CTA tile needs; its tensor memory receives the 128x256
// half of the accumulator that belongs to its A rows.  One elected thread of the even CTA issues the MMAs for
// the pair.
//
// Barrier plumbing (s = stage, b = accumulator buffer):
//   full[s]       lives in the leader; 1 arrival (leader's expect_tx for both CTAs' bytes) + the bytes of all four
//                 TMA loads (the odd CTA's loads name the leader's barrier through its cluster address)
//   empty[s]      one per CTA; tcgen05.commit with a 2-CTA multicast mask frees the stage in both
//   tmem_full[b]  one per CTA; same multicast commit after the last k-step of a tile
//   tmem_empty[b] lives in the leader; 8 arrivals = 4 epilogue warps of each CTA (remote arrive from the odd one)
// No TMA load carries a cluster multicast qualifier: every operand box is fetched by the CTA that uses it.
//
// Two variants fuse a tensor-parallel collective into the same kernel (FUSE template parameter):
//   FUSE_RS  GEMM → reduce-scatter: the epilogue stores every finished tile straight into the staging slot
//            [this rank] of the GPU that owns those output rows (plain peer stores over NVLink), remote chunks
//            first, so the transfer of tile i overlaps the math of tile i+1; the owner then sums its tp slots.
//   FUSE_AG  all-gather → GEMM: a few extra CTAs of the same launch pull the peers' activation shards into the
//            local gathered A matrix (plain peer loads) and bump a per-chunk ready counter; the TMA producers
//            order their tiles local-chunk-first and wait (bounded) for a chunk's counter before loading from it.
// All waits are bounded (common.cuh); both CTAs always meet at a cluster barrier before TMEM is released.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace tk {
namespace g2 {

constexpr int TM = 256, TN = 256, BK = 64, UMMA_K = 16, STAGES = 6;
constexpr int HALF_M = 128, HALF_N = 128;
constexpr int A_BYTES = HALF_M * BK * 2, B_BYTES = HALF_N * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;  // 32 KB per CTA
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int GROUP_M = 8;

constexpr int FUSE_NONE = 0, FUSE_RS = 1, FUSE_AG = 2, FUSE_STAGED = 3;  // STAGED: plain GEMM, bf16 output written through the staged epilogue
constexpr int FUSE_HS = 4;  // head scatter: fused q|k|v projection whose epilogue performs the Ulysses sequence→head exchange
constexpr int MAX_TP = 8;

struct Params {
  void* out;
  int M, N, K, ldo, out_fp32, accumulate;
  int* err;
  // tensor-parallel fusion
  int tp, rank, rows_per_rank;     // M = tp · rows_per_rank
  void* peer[MAX_TP];              // FUSE_RS: staging base [tp, rows_per_rank, N] of every rank; FUSE_AG: x shard of every rank
  void* gathered;                  // FUSE_AG: local [M, K] matrix the copier CTAs fill (the A operand)
  int* ready;                      // FUSE_AG: per-chunk counters, monotonically increasing across calls
  int ready_target;                // FUSE_AG: value a chunk's counter reaches when all copiers finished it in this call
  int copy_ctas;                   // FUSE_AG: CTAs [0, copy_ctas) copy (even number), the rest compute in pairs
  // FUSE_HS: the N columns are [q | k | v] in blocks of 128; peer c owns q blocks [c·qb/tp, (c+1)·qb/tp) and the same
  // share of the k and of the v blocks.  peer[c] = its buffer [tp·rows_per_rank, hs_ld]; this rank fills rows
  // [rank·rows_per_rank, +M) with the peer's blocks packed as [q_local | k_local | v_local].
  int hs_q_blocks, hs_kv_blocks, hs_ld;
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// Bounded wait until chunk `c` of the gathered matrix is complete.
__device__ __forceinline__ bool wait_chunk(const Params& p, int c) {
  const int* flag = p.ready + c;
  if (ld_acquire_gpu(flag) >= p.ready_target) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 0;; ++it) {
    if (ld_acquire_gpu(flag) >= p.ready_target) return true;
    if ((it & 0xff) == 0xff) {
      if (global_timer_ns() - t0 > 2000000000ull) { atomicCAS(p.err, 0, ERR_PEER_FLAG); return false; }
      if (*reinterpret_cast<volatile int*>(p.err) != 0) return false;
    }
  }
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load whose completion bytes go to a barrier that may sit in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs of the pair once the issued MMAs retire.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

template <int FUSE>
__device__ __forceinline__ bool tile_coord(const Params& p, int tile, int& m0, int& n0) {
  const int num_m = (p.M + TM - 1) / TM, num_n = (p.N + TN - 1) / TN;
  if (tile >= num_m * num_n) return false;
  const int per_group = GROUP_M * num_n;
  const int g = tile / per_group, first_m = g * GROUP_M;
  const int gsize = min(num_m - first_m, GROUP_M);
  const int r = tile - g * per_group;
  int mt = first_m + r % gsize;
  if constexpr (FUSE == FUSE_RS || FUSE == FUSE_AG) {
    // walk the row chunks in ring order: FUSE_RS sends remote chunks first and keeps its own for last,
    // FUSE_AG starts on its own chunk while the copiers fetch the others in the same order
    const int tiles_per_chunk = p.rows_per_rank / TM;
    const int pos = mt / tiles_per_chunk, within = mt - pos * tiles_per_chunk;
    const int c = (p.rank + pos + (FUSE == FUSE_RS ? 1 : 0)) % p.tp;
    mt = c * tiles_per_chunk + within;
  }
  m0 = mt * TM;
  n0 = (r / gsize) * TN;
  return true;
}

template <bool A_MN, bool B_MN, int FUSE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmL,
                         const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  // the reduce-scatter variant gives its sixth stage to the epilogue as a staging area for coalesced peer stores
  constexpr int NST = (FUSE == FUSE_RS || FUSE == FUSE_STAGED || FUSE == FUSE_HS) ? STAGES - 1 : STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader of the pair
  const int first_gemm = (FUSE == FUSE_AG) ? p.copy_ctas : 0;
  const int pair = (static_cast<int>(blockIdx.x) - first_gemm) >> 1;
  const int num_pairs = (static_cast<int>(gridDim.x) - first_gemm) >> 1;

  if constexpr (FUSE == FUSE_AG) {
    if (static_cast<int>(blockIdx.x) < p.copy_ctas) {
      // ------------------------------------------------------ copier CTAs: pull the shards, chunk by chunk
      // (lowest block indices, so they are resident before the compute CTAs that wait for them)
      // One thread drives a ring of 32 KB bulk copies (peer global → shared → local global): plain loads cannot keep
      // enough bytes in flight to cover the NVLink round trip, 6 x 32 KB per CTA can.
      if (threadIdx.x == 0) {
        constexpr uint32_t PIECE = STAGE_BYTES;  // 32 KB
        for (int s_ = 0; s_ < STAGES; ++s_) mbar_init(&full_bar[s_], 1);
        fence_barrier_init();
        fence_proxy_async_all();
        const int ncopy = p.copy_ctas, me = blockIdx.x;
        const long chunk_bytes = static_cast<long>(p.rows_per_rank) * p.K * 2;
        const long pieces = (chunk_bytes + PIECE - 1) / PIECE;
        uint32_t issued = 0, done = 0;  // pieces issued / stored by this CTA over all chunks (ring position = n % STAGES)
        bool ok = true;
        for (int pos = 1; ok && pos < p.tp; ++pos) {  // the local shard is read in place by the compute CTAs
          const int c = (p.rank + pos) % p.tp;
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.peer[c]);
          uint8_t* dst = reinterpret_cast<uint8_t*>(p.gathered) + static_cast<long>(c) * chunk_bytes;
          const long mine = me < pieces ? (pieces - me + ncopy - 1) / ncopy : 0;  // pieces me, me+ncopy, …
          long li = 0, si = 0;                                                    // next piece to load / to store
          while (si < mine) {
            // keep STAGES-1 loads in flight; the stage being refilled was stored one iteration ago
            while (li < mine && li - si < STAGES - 1) {
              const long off = (me + li * ncopy) * static_cast<long>(PIECE);
              const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long>(PIECE), chunk_bytes - off));
              const int st = issued % STAGES;
              asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // all but the newest store have left shared memory
              mbar_expect_tx(&full_bar[st], bytes);
              asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                           ::"r"(smem_u32(smem + st * PIECE)), "l"(src + off), "r"(bytes), "r"(smem_u32(&full_bar[st])) : "memory");
              ++issued; ++li;
            }
            const int st = done % STAGES;
            if (!mbar_wait(&full_bar[st], (done / STAGES) & 1, p.err, ERR_PEER_FLAG)) { ok = false; break; }
            const long off = (me + si * ncopy) * static_cast<long>(PIECE);
            const uint32_t bytes = static_cast<uint32_t>(min(static_cast<long>(PIECE), chunk_bytes - off));
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(dst + off), "r"(smem_u32(smem + st * PIECE)), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            ++done; ++si;
          }
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");         // my part of chunk c is written
          fence_proxy_async_all();
          __threadfence();
          if (ok) atomicAdd(p.ready + c, 1);
        }
      }
      return;  // a copier cluster holds copiers only: nothing of the pair protocol below concerns it
    }
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if constexpr (FUSE == FUSE_AG) tma_prefetch_desc(&tmL);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 8);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything can signal them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------------------------------------ producer (one per CTA)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int m0, n0;
      bool ok = true;
      for (int tile = pair; ok && tile_coord<FUSE>(p, tile, m0, n0); tile += num_pairs) {
        const int am = m0 + static_cast<int>(cta) * HALF_M, bn = n0 + static_cast<int>(cta) * HALF_N;
        const CUtensorMap* mapA = &tmA;
        int a_row = am;
        if constexpr (FUSE == FUSE_AG) {
          const int c = m0 / p.rows_per_rank;
          if (c == p.rank) {  // own shard: straight from where it already lives
            mapA = &tmL;
            a_row = am - c * p.rows_per_rank;
          } else {
            if (!wait_chunk(p, c)) { ok = false; break; }
            fence_proxy_async_all();  // the copiers' writes are ordered before this thread's TMA reads
          }
        }
        for (int k0 = 0; k0 < p.K; k0 += BK) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.err, ERR_PRODUCER_WAIT)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, mapA, bar, k0, a_row);                              // box {64 K, 128 rows}
          } else {
#pragma unroll
            for (int j = 0; j < HALF_M / 64; ++j) tma_load_2d_pair(sa + j * (64 * BK * 2), &tmA, bar, am + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmB, bar, k0, bn);
          } else {
#pragma unroll
            for (int j = 0; j < HALF_N / 64; ++j) tma_load_2d_pair(sb + j * (64 * BK * 2), &tmB, bar, bn + j * 64, k0);
          }
          if (++stage == NST) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok && cta == 0) {
        for (int s = 0; s < NST; ++s) mbar_wait(&full_bar[s], 0, nullptr, 0);  // bounded drain of copies in flight
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(TM, TN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0, acc = 0, acc_phase = 0;
      int m0, n0;
      bool ok = true;
      for (int tile = pair; ok && tile_coord<FUSE>(p, tile, m0, n0); tile += num_pairs) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.err, ERR_MMA_WAIT_TMEM)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        uint32_t first = 1;
        for (int k0 = 0; k0 < p.K; k0 += BK) {
          if (!mbar_wait(&full_bar[stage], phase, p.err, ERR_MMA_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = A_MN ? umma_desc(sa + k * (UMMA_K * 128), 64 * BK * 2, 1024) : umma_desc(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = B_MN ? umma_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024) : umma_desc(sb + k * (UMMA_K * 2), 16, 1024);
            umma_bf16_pair(d_tmem, ad, bd, idesc, first ? 0u : 1u);
            first = 0;
          }
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == NST) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    int m0, n0;
    bool ok = true;
    for (int tile = pair; ok && tile_coord<FUSE>(p, tile, m0, n0); tile += num_pairs) {
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.err, ERR_EPI_WAIT)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + static_cast<int>(cta) * HALF_M + q * 32 + lane;
      const bool row_ok = row < p.M;
      size_t out_row = static_cast<size_t>(row);
      void* out_base = p.out;
      if constexpr (FUSE == FUSE_RS) {
        // rows of chunk c belong to rank c: write them into slot [this rank] of that GPU's staging buffer
        const int c = min(row / p.rows_per_rank, p.tp - 1);
        out_base = p.peer[c];
        out_row = static_cast<size_t>(p.rank) * p.rows_per_rank + (row - c * p.rows_per_rank);
      }
      if constexpr (FUSE == FUSE_RS || FUSE == FUSE_STAGED || FUSE == FUSE_HS) {
        // Stage 32 rows x 128 columns (bf16) per warp in shared memory, then let every half-warp store one whole
        // 256-byte row segment: NVLink (and the local memory system) sees long contiguous writes instead of 64-byte
        // pieces of 32 different rows.
        uint8_t* stg = smem + (STAGES - 1) * STAGE_BYTES + q * 8192;
        const int row0 = m0 + static_cast<int>(cta) * HALF_M + q * 32;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            tmem_ld32(tmem_base + acc * TN + (half * 4 + cc) * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int chunk = (cc * 4 + j) ^ (lane & 15);
              *reinterpret_cast<uint4*>(stg + lane * 256 + chunk * 16) =
                  make_uint4(pack_bf16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])), pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                             pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])), pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
            }
          }
          __syncwarp();
          const int j = lane & 15;
          const int col = n0 + half * 128 + j * 8;
          int hs_peer = 0, hs_col = 0;
          if constexpr (FUSE == FUSE_HS) {
            // which peer owns this block of 128 columns, and where it sits in that peer's packed [q | k | v] row
            const int b = n0 / 128 + half, qb = p.hs_q_blocks, kb = p.hs_kv_blocks, qpl = qb / p.tp, kpl = kb / p.tp;
            int db;
            if (b < qb) { hs_peer = b / qpl; db = b - hs_peer * qpl; }
            else if (b < qb + kb) { const int bb = b - qb; hs_peer = bb / kpl; db = qpl + bb - hs_peer * kpl; }
            else { const int bb = b - qb - kb; hs_peer = bb / kpl; db = qpl + kpl + bb - hs_peer * kpl; }
            hs_peer = min(hs_peer, p.tp - 1);  // blocks past N are never stored (column check below)
            hs_col = db * 128 + j * 8;
          }
#pragma unroll 4
          for (int it = 0; it < 16; ++it) {
            const int lr = it * 2 + (lane >> 4);
            const int grow = row0 + lr;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + lr * 256 + ((j ^ (lr & 15)) * 16));
            if (grow < p.M && col + 8 <= p.N) {
              __nv_bfloat16* o;
              if constexpr (FUSE == FUSE_RS) {
                const int c = min(grow / p.rows_per_rank, p.tp - 1);
                o = reinterpret_cast<__nv_bfloat16*>(p.peer[c]) +
                    (static_cast<size_t>(p.rank) * p.rows_per_rank + (grow - c * p.rows_per_rank)) * p.ldo + col;
              } else if constexpr (FUSE == FUSE_HS) {
                o = reinterpret_cast<__nv_bfloat16*>(p.peer[hs_peer]) + (static_cast<size_t>(p.rank) * p.rows_per_rank + grow) * p.hs_ld + hs_col;
              } else {
                o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(grow) * p.ldo + col;
              }
              *reinterpret_cast<uint4*>(o) = v;
            }
          }
          __syncwarp();
        }
      } else
#pragma unroll 1
      for (int c = 0; c < TN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * TN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        if (p.out_fp32) {
          float* o = reinterpret_cast<float*>(out_base) + out_row * p.ldo + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (col0 + j + 4 <= p.N) {
              float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              if (p.accumulate) {
                const float4 old = *reinterpret_cast<float4*>(o + j);
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
              }
              *reinterpret_cast<float4*>(o + j) = v;
            } else {
              for (int jj = j; jj < j + 4 && col0 + jj < p.N; ++jj) o[jj] = __uint_as_float(r[jj]) + (p.accumulate ? o[jj] : 0.f);
            }
          }
        } else {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out_base) + out_row * p.ldo + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j + 8 <= p.N) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j + e]);
              if (p.accumulate) {
                const uint4 old = *reinterpret_cast<uint4*>(o + j);
                const float2 a0 = unpack_bf16(old.x), a1 = unpack_bf16(old.y), a2 = unpack_bf16(old.z), a3 = unpack_bf16(old.w);
                f[0] += a0.x; f[1] += a0.y; f[2] += a1.x; f[3] += a1.y;
                f[4] += a2.x; f[5] += a2.y; f[6] += a3.x; f[7] += a3.y;
              }
              *reinterpret_cast<uint4*>(o + j) = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
            } else {
              for (int jj = j; jj < j + 8 && col0 + jj < p.N; ++jj)
                o[jj] = __float2bfloat16(__uint_as_float(r[jj]) + (p.accumulate ? __bfloat162float(o[jj]) : 0.f));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody in the pair touches the other's shared or tensor memory after this point
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace g2

// Number of SM pairs that can be resident at once for this kernel (cached per device); 0 when clusters cannot launch.
template <typename Kern>
static int max_pairs(Kern kern) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(num_sms() & ~1, 1, 1);
  cfg.blockDim = dim3(g2::THREADS, 1, 1);
  cfg.dynamicSmemBytes = g2::SMEM_BYTES;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// 1: bf16 outputs go through the shared-memory staged epilogue (5 operand stages); 0: direct stores (6 stages).
static int g_staged_epilogue = [] {
  const char* e = getenv("TK_GEMM_STAGED");
  return e ? atoi(e) : 1;
}();
void set_gemm_staged(int64_t v) { g_staged_epilogue = static_cast<int>(v); }

// Dense GEMM on SM pairs; same contract as the single-CTA path.  Returns false when the shape is not eligible
// (the caller then uses the single-CTA kernel).
bool gemm_pair_launch(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, void* out, int M, int N, int K, int ldo,
                      bool out_fp32, bool accumulate, cudaStream_t stream) {
  g2::Params p{};
  p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.out_fp32 = out_fp32 ? 1 : 0; p.accumulate = accumulate ? 1 : 0; p.err = error_word();
  const int tiles = ((M + g2::TM - 1) / g2::TM) * ((N + g2::TN - 1) / g2::TN);
#define TK_LAUNCH2(AM, BMN)                                                                                            \
  do {                                                                                                                 \
    static int pairs = -1;                                                                                             \
    auto kern = g2::gemm_tcgen05_pair_kernel<AM, BMN, g2::FUSE_NONE>;                                                                 \
    if (pairs < 0) {                                                                                                   \
      TK_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, g2::SMEM_BYTES));          \
      pairs = max_pairs(kern);                                                                                         \
    }                                                                                                                  \
    if (pairs <= 0) return false;                                                                                      \
    const int grid = 2 * std::min(tiles, std::min(pairs, num_sms() / 2));                                              \
    kern<<<grid, g2::THREADS, g2::SMEM_BYTES, stream>>>(ta, tb, ta, p);                                                \
  } while (0)
#define TK_LAUNCH2S(AM, BMN)                                                                                           \
  do {                                                                                                                 \
    static int pairs = -1;                                                                                             \
    auto kern = g2::gemm_tcgen05_pair_kernel<AM, BMN, g2::FUSE_STAGED>;                                                \
    if (pairs < 0) {                                                                                                   \
      TK_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, g2::SMEM_BYTES));          \
      pairs = max_pairs(kern);                                                                                         \
    }                                                                                                                  \
    if (pairs <= 0) return false;                                                                                      \
    const int grid = 2 * std::min(tiles, std::min(pairs, num_sms() / 2));                                              \
    kern<<<grid, g2::THREADS, g2::SMEM_BYTES, stream>>>(ta, tb, ta, p);                                                \
  } while (0)
  const bool staged = g_staged_epilogue && !out_fp32 && !accumulate && N % 8 == 0;
  if (staged) {
    if (!a_mn && !b_mn) TK_LAUNCH2S(false, false);
    else if (!a_mn && b_mn) TK_LAUNCH2S(false, true);
    else if (a_mn && b_mn) TK_LAUNCH2S(true, true);
    else return false;
  } else {
    if (!a_mn && !b_mn) TK_LAUNCH2(false, false);
    else if (!a_mn && b_mn) TK_LAUNCH2(false, true);
    else if (a_mn && b_mn) TK_LAUNCH2(true, true);
    else return false;
  }
#undef TK_LAUNCH2S
#undef TK_LAUNCH2
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return true;
}


// ------------------------------------------------------------------------------------------------ fused TP paths
static void check_bf16_2d(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 2 && t.is_contiguous(), name, " must be a contiguous 2-D bf16 CUDA tensor");
  TORCH_CHECK(t.size(1) % 8 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, ": rows must be 16-byte multiples");
}

template <int FUSE>
static void launch_fused(bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tl, const g2::Params& p, int copy_ctas,
                         cudaStream_t stream) {
  const int tiles = ((p.M + g2::TM - 1) / g2::TM) * ((p.N + g2::TN - 1) / g2::TN);
#define TK_LAUNCH_F(BMN)                                                                                               \
  do {                                                                                                                 \
    static int pairs = -1;                                                                                             \
    auto kern = g2::gemm_tcgen05_pair_kernel<false, BMN, FUSE>;                                                        \
    if (pairs < 0) {                                                                                                   \
      TK_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, g2::SMEM_BYTES));          \
      pairs = max_pairs(kern);                                                                                         \
    }                                                                                                                  \
    TORCH_CHECK(pairs > copy_ctas / 2, "SM-pair kernel cannot be resident on this device");                           \
    const int avail = std::min(pairs, num_sms() / 2) - copy_ctas / 2;                                                  \
    const int grid = copy_ctas + 2 * std::min(tiles, avail);                                                           \
    kern<<<grid, g2::THREADS, g2::SMEM_BYTES, stream>>>(ta, tb, tl, p);                                                \
  } while (0)
  if (b_mn) TK_LAUNCH_F(true); else TK_LAUNCH_F(false);
#undef TK_LAUNCH_F
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
}

// Row-parallel linear with the reduce-scatter in the epilogue.  a [T, Kl] (this rank's K slice of the activations),
// w [N, Kl] ('nt') or [Kl, N] ('nn').  Tile rows of chunk c are stored into slot [rank] of rank c's staging buffer
// (`stage_ptrs[c]`, layout [tp, T/tp, N] bf16).  The caller passes a cross-GPU barrier and sums its own slots.
void gemm_rs(const torch::Tensor& a, const torch::Tensor& w, const std::string& layout, const std::vector<int64_t>& stage_ptrs, int64_t rank) {
  check_bf16_2d(a, "a");
  check_bf16_2d(w, "w");
  const int tp = stage_ptrs.size();
  TORCH_CHECK(tp >= 1 && tp <= g2::MAX_TP, "tp out of range");
  const bool b_mn = layout == "nn";
  TORCH_CHECK(b_mn || layout == "nt", "layout must be nt|nn");
  const int M = a.size(0), K = a.size(1), N = b_mn ? w.size(1) : w.size(0);
  TORCH_CHECK((b_mn ? w.size(0) : w.size(1)) == K, "K mismatch");
  TORCH_CHECK(M % tp == 0 && (M / tp) % g2::TM == 0, "rows per rank must be a multiple of ", g2::TM);
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "K and N must be multiples of 8");
  c10::cuda::CUDAGuard guard(a.device());
  CUtensorMap ta = make_tmap_2d(a.data_ptr(), K, M, a.stride(0), g2::BK, 128);
  CUtensorMap tb = b_mn ? make_tmap_2d(w.data_ptr(), w.size(1), w.size(0), w.stride(0), 64, g2::BK)
                        : make_tmap_2d(w.data_ptr(), w.size(1), w.size(0), w.stride(0), g2::BK, 128);
  g2::Params p{};
  p.out = nullptr; p.M = M; p.N = N; p.K = K; p.ldo = N; p.out_fp32 = 0; p.accumulate = 0; p.err = error_word();
  p.tp = tp; p.rank = static_cast<int>(rank); p.rows_per_rank = M / tp;
  for (int i = 0; i < tp; ++i) p.peer[i] = reinterpret_cast<void*>(stage_ptrs[i]);
  launch_fused<g2::FUSE_RS>(b_mn, ta, tb, ta, p, 0, at::cuda::getCurrentCUDAStream());
}

// Fused q|k|v projection with the Ulysses sequence→head exchange in the epilogue.  x [T_local, K], w [N, K] with
// N = (q_blocks + 2·kv_blocks)·128 laid out [q | k | v].  `dest_ptrs[c]` = rank c's buffer [sp·rows_per_rank, N/sp] bf16
// (symmetric memory); this rank writes rows [rank·rows_per_rank, +T_local) of every peer's buffer.  The caller brackets
// the call with cross-GPU barriers (buffers free before, pushes landed after).
void gemm_head_scatter(const torch::Tensor& x, const torch::Tensor& w, const std::vector<int64_t>& dest_ptrs, int64_t rank, int64_t rows_per_rank,
                       int64_t q_blocks, int64_t kv_blocks) {
  check_bf16_2d(x, "x");
  check_bf16_2d(w, "w");
  const int sp = dest_ptrs.size();
  TORCH_CHECK(sp >= 1 && sp <= g2::MAX_TP, "group size out of range");
  TORCH_CHECK(rank >= 0 && rank < sp, "rank out of range");
  const int M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "K mismatch");
  TORCH_CHECK(q_blocks > 0 && kv_blocks > 0 && q_blocks % sp == 0 && kv_blocks % sp == 0, "q and kv column blocks must divide over the group");
  TORCH_CHECK(N == (q_blocks + 2 * kv_blocks) * 128, "w rows must be (q_blocks + 2 kv_blocks) * 128");
  TORCH_CHECK(M <= rows_per_rank, "more rows than a rank's share of the destination");
  TORCH_CHECK(K % 8 == 0, "K must be a multiple of 8");
  for (int i = 0; i < sp; ++i) TORCH_CHECK(dest_ptrs[i] % 16 == 0, "destination buffers must be 16-byte aligned");
  if (M == 0) return;
  c10::cuda::CUDAGuard guard(x.device());
  CUtensorMap ta = make_tmap_2d(x.data_ptr(), K, M, x.stride(0), g2::BK, 128);
  CUtensorMap tb = make_tmap_2d(w.data_ptr(), w.size(1), w.size(0), w.stride(0), g2::BK, 128);
  g2::Params p{};
  p.out = nullptr; p.M = M; p.N = N; p.K = K; p.ldo = N; p.out_fp32 = 0; p.accumulate = 0; p.err = error_word();
  p.tp = sp; p.rank = static_cast<int>(rank); p.rows_per_rank = static_cast<int>(rows_per_rank);
  for (int i = 0; i < sp; ++i) p.peer[i] = reinterpret_cast<void*>(dest_ptrs[i]);
  p.hs_q_blocks = static_cast<int>(q_blocks); p.hs_kv_blocks = static_cast<int>(kv_blocks); p.hs_ld = N / sp;
  launch_fused<g2::FUSE_HS>(false, ta, tb, ta, p, 0, at::cuda::getCurrentCUDAStream());
}

// Column-parallel linear with the all-gather in the prologue.  `x_ptrs[c]` = rank c's [rows_per_rank, K] bf16 shard
// (symmetric memory); returns {y [tp·rows_per_rank, N], gathered [tp·rows_per_rank, K]}.  `ready` holds tp int32
// counters that only ever grow: every call adds copy_ctas to each and waits for `ready_target` = the new total.
std::vector<torch::Tensor> gemm_ag(const std::vector<int64_t>& x_ptrs, int64_t rows_per_rank, const torch::Tensor& w, const std::string& layout,
                                   int64_t rank, const torch::Tensor& ready, int64_t ready_target, int64_t copy_ctas) {
  check_bf16_2d(w, "w");
  const int tp = x_ptrs.size();
  TORCH_CHECK(tp >= 1 && tp <= g2::MAX_TP, "tp out of range");
  TORCH_CHECK(ready.is_cuda() && ready.scalar_type() == torch::kInt32 && ready.numel() >= tp && ready.is_contiguous(), "ready: int32 [tp]");
  TORCH_CHECK(copy_ctas >= 2 && copy_ctas % 2 == 0 && copy_ctas <= 64, "copy_ctas must be even, 2..64");
  const bool b_mn = layout == "nn";
  TORCH_CHECK(b_mn || layout == "nt", "layout must be nt|nn");
  const int K = b_mn ? w.size(0) : w.size(1), N = b_mn ? w.size(1) : w.size(0);
  TORCH_CHECK(rows_per_rank % g2::TM == 0, "rows per rank must be a multiple of ", g2::TM);
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "K and N must be multiples of 8");
  TORCH_CHECK(ready_target > 0 && ready_target < (1ll << 30), "ready counters exhausted: reset them");
  c10::cuda::CUDAGuard guard(w.device());
  const int M = tp * static_cast<int>(rows_per_rank);
  auto gathered = torch::empty({M, K}, w.options());
  auto out = torch::empty({M, N}, w.options());
  CUtensorMap ta = make_tmap_2d(gathered.data_ptr(), K, M, K, g2::BK, 128);
  CUtensorMap tb = b_mn ? make_tmap_2d(w.data_ptr(), w.size(1), w.size(0), w.stride(0), 64, g2::BK)
                        : make_tmap_2d(w.data_ptr(), w.size(1), w.size(0), w.stride(0), g2::BK, 128);
  g2::Params p{};
  p.out = out.data_ptr(); p.M = M; p.N = N; p.K = K; p.ldo = N; p.out_fp32 = 0; p.accumulate = 0; p.err = error_word();
  p.tp = tp; p.rank = static_cast<int>(rank); p.rows_per_rank = static_cast<int>(rows_per_rank);
  for (int i = 0; i < tp; ++i) p.peer[i] = reinterpret_cast<void*>(x_ptrs[i]);
  p.gathered = gathered.data_ptr(); p.ready = ready.data_ptr<int>(); p.ready_target = static_cast<int>(ready_target);
  p.copy_ctas = static_cast<int>(copy_ctas);
  // the rank's own shard: read in place by the compute CTAs, and copied into `gathered` for the caller's wgrad
  CUtensorMap tl = make_tmap_2d(reinterpret_cast<void*>(x_ptrs[rank]), K, rows_per_rank, K, g2::BK, 128);
  TK_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(gathered.data_ptr()) + rank * rows_per_rank * K * 2, reinterpret_cast<void*>(x_ptrs[rank]),
                                rows_per_rank * K * 2, cudaMemcpyDeviceToDevice, at::cuda::getCurrentCUDAStream()));
  launch_fused<g2::FUSE_AG>(b_mn, ta, tb, tl, p, static_cast<int>(copy_ctas), at::cuda::getCurrentCUDAStream());
  return {out, gathered};
}

// out[r, :] = Σ_s stage[s, r, :]  (fp32 sum of the tp staging slots, bf16 result)
__global__ void __launch_bounds__(256) stage_reduce_kernel(const uint4* __restrict__ stage, uint4* __restrict__ out, long vecs, int tp) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < vecs; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < tp; ++s) {
      const uint4 u = stage[static_cast<long>(s) * vecs + i];
      const uint32_t* q = &u.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16(q[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    out[i] = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

torch::Tensor tp_stage_reduce(const torch::Tensor& stage) {
  TORCH_CHECK(stage.is_cuda() && stage.scalar_type() == torch::kBFloat16 && stage.dim() == 3 && stage.is_contiguous(), "stage [tp, rows, N] bf16");
  c10::cuda::CUDAGuard guard(stage.device());
  const int tp = stage.size(0);
  auto out = torch::empty({stage.size(1), stage.size(2)}, stage.options());
  const long vecs = out.numel() / 8;
  TORCH_CHECK(out.numel() % 8 == 0, "rows·N must be a multiple of 8");
  if (vecs == 0) return out;
  const int grid = static_cast<int>(std::min<long>((vecs + 255) / 256, static_cast<long>(num_sms()) * 8));
  stage_reduce_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(reinterpret_cast<const uint4*>(stage.data_ptr()),
                                                                          reinterpret_cast<uint4*>(out.data_ptr()), vecs, tp);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
  return out;
}

}  // namespace tk
