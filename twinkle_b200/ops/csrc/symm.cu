// Peer-memory (NVLink / NVSwitch) data plane: symmetric buffers shared through CUDA IPC and the
// kernels that move data between GPUs with plain peer loads / stores.
//
//   symm_alloc / symm_open          one cudaMalloc per symmetric buffer, handle exchanged by the host
//   symm_barrier                    cross-GPU barrier: every rank writes an epoch into each peer's flag
//                                   slot (st.release.sys) and waits for all slots (ld.acquire.sys, bounded)
//   peer_all_gather                 pull: out[k] = peer_k.shard for every k (16-byte peer loads)
//   peer_pull                       strided pull of rows × chunk bytes per (peer, section) job, 8 loads in flight
//                                   per thread: Ulysses head↔sequence exchange, parameter all-gather
//   peer_reduce_scatter_acc         pull: grad_shard += scale · Σ_k peer_k.full[rank slice]  (bf16 → fp32,
//                                   cast + scale + accumulate fused; optional Σg² partial)
//   peer_all_to_all_heads           Ulysses head↔sequence exchange: each rank pushes its slices straight
//                                   into the destination layout of the peers
//   peer_copy_cast                  trainer → sampler weight push with optional fp32→bf16 cast
//
// No TMA multicast and no library kernel ever touches a peer pointer; every wait is bounded and reports
// through the error word.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "common.cuh"
#include "host.h"

namespace py = pybind11;

namespace tk {

using bf16 = __nv_bfloat16;
constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

// ------------------------------------------------------------ allocation
// Returns (uint8 tensor over the new allocation, IPC handle, byte offset of the allocation inside the
// driver block the handle refers to).  cudaMalloc may carve small requests out of a larger block and the
// IPC handle always maps the whole block, so the opener must add this offset to the mapped base.
std::tuple<torch::Tensor, py::bytes, int64_t> symm_alloc(int64_t nbytes) {
  int dev = 0;
  TK_CUDA_CHECK(cudaGetDevice(&dev));
  void* ptr = nullptr;
  const int64_t gran = 2 << 20;  // whole 2 MiB pages: every symmetric buffer owns its driver block
  nbytes = (nbytes + gran - 1) / gran * gran;
  cudaError_t rc = cudaMalloc(&ptr, nbytes);
  if (rc == cudaErrorMemoryAllocation) {
    // Symmetric buffers come straight from the driver, next to PyTorch's caching allocator.  Blocks that the allocator
    // holds but does not use are handed back and the request is made once more; the failed attempt's error code is
    // cleared so that it does not surface in an unrelated later call.
    (void)cudaGetLastError();
    TK_CUDA_CHECK(cudaDeviceSynchronize());
    c10::cuda::CUDACachingAllocator::emptyCache();
    rc = cudaMalloc(&ptr, nbytes);
    if (rc != cudaSuccess) (void)cudaGetLastError();
  }
  TORCH_CHECK(rc == cudaSuccess, "symmetric allocation of ", nbytes, " bytes failed: ", cudaGetErrorString(rc));
  TK_CUDA_CHECK(cudaMemset(ptr, 0, nbytes));
  TK_CUDA_CHECK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  TK_CUDA_CHECK(cudaIpcGetMemHandle(&h, ptr));
  int64_t offset = 0;
  {
    using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) == cudaSuccess && fn != nullptr) {
      CUdeviceptr base = 0;
      size_t size = 0;
      if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) == CUDA_SUCCESS)
        offset = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
    }
  }
  auto t = torch::from_blob(ptr, {nbytes}, [](void* p) { cudaFree(p); }, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, dev));
  return {t, py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)), offset};
}

int64_t symm_open(const py::bytes& handle) {
  std::string s = handle;
  TORCH_CHECK(s.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  cudaIpcMemHandle_t h;
  memcpy(&h, s.data(), sizeof(h));
  void* ptr = nullptr;
  TK_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return reinterpret_cast<int64_t>(ptr);
}

void symm_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

// ----------------------------------------------------------------- barrier
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags: each rank owns int[MAX_PEERS]; slot k of rank r is written by rank k.
__global__ void symm_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, int* err, unsigned long long limit_ns) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.p[t]) + rank, epoch);
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + t;
    // once any wait has failed on this device, later barriers do not wait at all: the step is already
    // lost and the host raises on its next check of the error word
    if (*reinterpret_cast<volatile int*>(err) != 0) return;
    const uint64_t t0 = global_timer_ns();
    uint32_t it = 0;
    while (ld_acquire_sys(mine) < epoch) {
      if ((++it & 0xff) == 0) {
        if (global_timer_ns() - t0 > limit_ns) {  // default 3 s
          atomicCAS(err, 0, ERR_PEER_FLAG);
          break;
        }
        if (*reinterpret_cast<volatile int*>(err) != 0) break;
      }
    }
  }
}

void symm_barrier(const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t epoch, int64_t timeout_ms) {
  PeerPtrs f{};
  const int world = flag_ptrs.size();
  TORCH_CHECK(world <= MAX_PEERS, "too many peers");
  for (int i = 0; i < world; ++i) f.p[i] = reinterpret_cast<void*>(flag_ptrs[i]);
  symm_barrier_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(f, static_cast<int>(rank), world, static_cast<int>(epoch), error_word(),
                                                                      static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 3000) * 1000000ull);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
}

// --------------------------------------------------------------- all-gather
// grid.y = source rank; each block copies a contiguous stripe with 16-byte accesses.
__global__ void peer_all_gather_kernel(uint4* __restrict__ out, PeerPtrs shards, long shard_vecs, int rank, int skip_self) {
  const int src = blockIdx.y;
  if (skip_self && src == rank) return;
  const uint4* in = reinterpret_cast<const uint4*>(shards.p[src]);
  uint4* dst = out + static_cast<long>(src) * shard_vecs;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < shard_vecs; i += static_cast<long>(gridDim.x) * blockDim.x)
    dst[i] = in[i];
}

void peer_all_gather(torch::Tensor out, const std::vector<int64_t>& shard_ptrs, int64_t shard_bytes, int64_t rank, int64_t blocks_per_peer) {
  const int world = shard_ptrs.size();
  TORCH_CHECK(world <= MAX_PEERS && shard_bytes % 16 == 0, "shard must be a multiple of 16 bytes");
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() * out.element_size() >= shard_bytes * world, "out too small");
  c10::cuda::CUDAGuard guard(out.device());
  PeerPtrs s{};
  for (int i = 0; i < world; ++i) s.p[i] = reinterpret_cast<void*>(shard_ptrs[i]);
  const bool aliased = reinterpret_cast<int64_t>(out.data_ptr()) + rank * shard_bytes == shard_ptrs[rank];
  dim3 grid(static_cast<unsigned>(blocks_per_peer), world);
  peer_all_gather_kernel<<<grid, 512, 0, at::cuda::getCurrentCUDAStream()>>>(reinterpret_cast<uint4*>(out.data_ptr()), s, shard_bytes / 16,
                                                                             static_cast<int>(rank), aliased ? 1 : 0);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
}


// ------------------------------------------------------------- strided pull
// The general receive-side copy of this file: a launch carries up to MAX_JOBS jobs, each "rows × chunk bytes from
// src (row stride src_stride) to dst (row stride dst_stride)".  The source of a job is usually another GPU's
// symmetric buffer; the destination is always local.  One job per (peer, tensor section) expresses the Ulysses
// head↔sequence exchange in both directions (a rank pulls exactly the head slice / token chunk it will own) and, with
// rows = 1, the parameter all-gather.  Every thread keeps UNROLL independent 16-byte loads in flight before it
// stores, which is what the NVLink round trip needs: with one load per thread in flight the same copy ran several
// times slower.  No shared memory is used, so the kernel can share SMs with a resident GEMM when it runs on a side
// stream.
constexpr int MAX_JOBS = 48;
struct PullJob {
  const uint8_t* src;
  uint8_t* dst;
  long src_stride, dst_stride;  // bytes between rows
  int chunk_vecs;               // 16-byte vectors per row
  int rows;
};
struct PullJobs {
  PullJob j[MAX_JOBS];
};

__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <int UNROLL>
__global__ void __launch_bounds__(512) peer_pull_kernel(const __grid_constant__ PullJobs jobs) {
  const PullJob& job = jobs.j[blockIdx.y];
  const long nvec = static_cast<long>(job.rows) * job.chunk_vecs;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  const int cv = job.chunk_vecs;
  for (long base = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; base < nvec; base += stride * UNROLL) {
    uint4 r[UNROLL];
    long doff[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long v = base + u * stride;
      if (v < nvec) {
        const long row = v / cv;
        const long c = (v - row * cv) << 4;
        r[u] = ld_global_v4(job.src + row * job.src_stride + c);
        doff[u] = row * job.dst_stride + c;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long v = base + u * stride;
      if (v < nvec) *reinterpret_cast<uint4*>(job.dst + doff[u]) = r[u];
    }
  }
}

// jobs: parallel lists (source address, destination address, source row stride, destination row stride, bytes per
// row, rows).  Addresses, strides and row sizes must be multiples of 16 bytes.
void peer_pull(const std::vector<int64_t>& src, const std::vector<int64_t>& dst, const std::vector<int64_t>& src_stride,
               const std::vector<int64_t>& dst_stride, const std::vector<int64_t>& chunk_bytes, const std::vector<int64_t>& rows,
               int64_t blocks_per_job) {
  const size_t n = src.size();
  TORCH_CHECK(n > 0 && n <= MAX_JOBS, "peer_pull: between 1 and ", MAX_JOBS, " jobs per launch");
  TORCH_CHECK(dst.size() == n && src_stride.size() == n && dst_stride.size() == n && chunk_bytes.size() == n && rows.size() == n,
              "peer_pull: job lists differ in length");
  PullJobs J{};
  long max_vecs = 0;
  for (size_t i = 0; i < n; ++i) {
    TORCH_CHECK(src[i] % 16 == 0 && dst[i] % 16 == 0 && src_stride[i] % 16 == 0 && dst_stride[i] % 16 == 0 && chunk_bytes[i] % 16 == 0,
                "peer_pull: addresses, strides and row sizes must be multiples of 16 bytes");
    TORCH_CHECK(chunk_bytes[i] / 16 < (1L << 31) && rows[i] < (1L << 31) && rows[i] >= 0, "peer_pull: job too large");
    J.j[i] = PullJob{reinterpret_cast<const uint8_t*>(src[i]), reinterpret_cast<uint8_t*>(dst[i]), static_cast<long>(src_stride[i]),
                     static_cast<long>(dst_stride[i]), static_cast<int>(chunk_bytes[i] / 16), static_cast<int>(rows[i])};
    max_vecs = std::max<long>(max_vecs, rows[i] * (chunk_bytes[i] / 16));
  }
  if (max_vecs == 0) return;
  constexpr int UNROLL = 8;
  const long want = (max_vecs + 512L * UNROLL - 1) / (512L * UNROLL);
  const unsigned bx = static_cast<unsigned>(std::max<long>(1, std::min<long>(want, blocks_per_job)));
  peer_pull_kernel<UNROLL><<<dim3(bx, static_cast<unsigned>(n)), 512, 0, at::cuda::getCurrentCUDAStream()>>>(J);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
}

// ----------------------------------------------------------- reduce-scatter
// grad_shard[i] += scale · Σ_k full_k[rank·n + i]; reads 8 bf16 per peer per step, accumulates in fp32.
__global__ void __launch_bounds__(512) peer_reduce_scatter_kernel(float* __restrict__ grad_shard, PeerPtrs fulls, long shard_numel, int rank, int world,
                                                                  float scale, float* __restrict__ sumsq) {
  constexpr int U = 4;  // vectors per thread per round: U × world 16-byte peer loads in flight before the first add
  const long nvec = shard_numel >> 3;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  float local_sq = 0.f;
  for (long v0 = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; v0 < nvec; v0 += stride * U) {
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
    // start with a different peer on every rank so the NVSwitch ports are loaded evenly
    for (int j = 0; j < world; ++j) {
      const int k = (rank + j) % world;
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(fulls.p[k]) + static_cast<long>(rank) * shard_numel);
      uint4 u4[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long v = v0 + u * stride;
        if (v < nvec) u4[u] = ld_global_v4(src + v);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long v = v0 + u * stride;
        if (v < nvec) {
          const uint32_t* pu = &u4[u].x;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = unpack_bf16(pu[q]);
            acc[u][2 * q] += f.x;
            acc[u][2 * q + 1] += f.y;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long v = v0 + u * stride;
      if (v >= nvec) continue;
      float4* g = reinterpret_cast<float4*>(grad_shard + v * 8);
      float4 a = g[0], b = g[1];
      a.x += acc[u][0] * scale; a.y += acc[u][1] * scale; a.z += acc[u][2] * scale; a.w += acc[u][3] * scale;
      b.x += acc[u][4] * scale; b.y += acc[u][5] * scale; b.z += acc[u][6] * scale; b.w += acc[u][7] * scale;
      g[0] = a; g[1] = b;
      if (sumsq) local_sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
    }
  }
  if (sumsq) {
    local_sq = warp_sum(local_sq);
    if ((threadIdx.x & 31) == 0) atomicAdd(sumsq, local_sq);
  }
}

void peer_reduce_scatter_acc(torch::Tensor grad_shard, const std::vector<int64_t>& full_ptrs, int64_t rank, double scale,
                             const c10::optional<torch::Tensor>& sumsq, int64_t blocks) {
  const int world = full_ptrs.size();
  TORCH_CHECK(grad_shard.is_cuda() && grad_shard.scalar_type() == torch::kFloat32 && grad_shard.is_contiguous(), "grad_shard fp32");
  TORCH_CHECK(grad_shard.numel() % 8 == 0, "shard size must be a multiple of 8");
  c10::cuda::CUDAGuard guard(grad_shard.device());
  PeerPtrs f{};
  for (int i = 0; i < world; ++i) f.p[i] = reinterpret_cast<void*>(full_ptrs[i]);
  peer_reduce_scatter_kernel<<<static_cast<unsigned>(blocks), 512, 0, at::cuda::getCurrentCUDAStream()>>>(
      grad_shard.data_ptr<float>(), f, grad_shard.numel(), static_cast<int>(rank), world, static_cast<float>(scale),
      (sumsq.has_value() && sumsq->defined()) ? sumsq->data_ptr<float>() : nullptr);
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
}

// ------------------------------------------------------- Ulysses all-to-all
// seq→head: local x [t, H, D] (this rank's token chunk, all heads) → peer j receives heads [j·hl, (j+1)·hl)
//           at rows [rank·t, (rank+1)·t) of its [sp·t, hl, D] buffer.            (push)
// head→seq: local x [sp·t, hl, D] → peer j receives token chunk j, placed at head offset rank·hl of its
//           [t, H, D] buffer.                                                      (push)
__global__ void ulysses_seq_to_head_kernel(const uint4* __restrict__ x, PeerPtrs outs, int t, int H, int hl, int rank, int vec_per_head) {
  // one block-stride loop over (token, head, vec)
  const long total = static_cast<long>(t) * H * vec_per_head;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec_per_head);
    const long th = i / vec_per_head;
    const int h = static_cast<int>(th % H), tok = static_cast<int>(th / H);
    const int dst_rank = h / hl, hloc = h - dst_rank * hl;
    uint4* dst = reinterpret_cast<uint4*>(outs.p[dst_rank]);
    dst[(static_cast<long>(rank) * t + tok) * hl * vec_per_head + static_cast<long>(hloc) * vec_per_head + v] = x[i];
  }
}
__global__ void ulysses_head_to_seq_kernel(const uint4* __restrict__ x, PeerPtrs outs, int t, int H, int hl, int rank, int sp, int vec_per_head) {
  const long total = static_cast<long>(sp) * t * hl * vec_per_head;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec_per_head);
    const long th = i / vec_per_head;
    const int hloc = static_cast<int>(th % hl);
    const long tokg = th / hl;
    const int dst_rank = static_cast<int>(tokg / t), tok = static_cast<int>(tokg % t);
    uint4* dst = reinterpret_cast<uint4*>(outs.p[dst_rank]);
    dst[(static_cast<long>(tok) * H + rank * hl + hloc) * vec_per_head + v] = x[i];
  }
}

void ulysses_exchange(const torch::Tensor& x, const std::vector<int64_t>& out_ptrs, int64_t rank, bool seq_to_head, int64_t heads_total) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 3, "x [tokens, heads, D] contiguous");
  const int sp = out_ptrs.size();
  const int D = x.size(2);
  TORCH_CHECK((D * x.element_size()) % 16 == 0, "head row must be a multiple of 16 bytes");
  c10::cuda::CUDAGuard guard(x.device());
  PeerPtrs o{};
  for (int i = 0; i < sp; ++i) o.p[i] = reinterpret_cast<void*>(out_ptrs[i]);
  const int vph = D * x.element_size() / 16;
  const long total = x.numel() * x.element_size() / 16;
  const int blocks = static_cast<int>(std::min<long>((total + 511) / 512, num_sms() * 4L));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (seq_to_head) {
    const int t = x.size(0), H = x.size(1);
    TORCH_CHECK(H % sp == 0, "heads must divide over the sequence-parallel group");
    ulysses_seq_to_head_kernel<<<blocks, 512, 0, stream>>>(reinterpret_cast<const uint4*>(x.data_ptr()), o, t, H, H / sp, static_cast<int>(rank), vph);
  } else {
    const int hl = x.size(1), t = x.size(0) / sp;
    ulysses_head_to_seq_kernel<<<blocks, 512, 0, stream>>>(reinterpret_cast<const uint4*>(x.data_ptr()), o, t, static_cast<int>(heads_total), hl,
                                                           static_cast<int>(rank), sp, vph);
  }
  count_launch();
  TK_CUDA_CHECK(cudaGetLastError());
}

// ------------------------------------------------------------ weight push
template <typename SrcT>
__global__ void peer_copy_cast_kernel(const SrcT* __restrict__ src, bf16* __restrict__ dst, long n) {
  for (long i = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) * 8; i < n; i += static_cast<long>(gridDim.x) * blockDim.x * 8) {
    if (i + 8 <= n) {
      uint4 o;
      if constexpr (std::is_same<SrcT, float>::value) {
        const float4 a = *reinterpret_cast<const float4*>(src + i), b = *reinterpret_cast<const float4*>(src + i + 4);
        o = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
      } else {
        o = *reinterpret_cast<const uint4*>(src + i);
      }
      *reinterpret_cast<uint4*>(dst + i) = o;
    } else {
      for (long j = i; j < n; ++j) {
        if constexpr (std::is_same<SrcT, float>::value) dst[j] = __float2bfloat16(src[j]); else dst[j] = src[j];
      }
    }
  }
}

// Copies `src` (bf16 or fp32, local) into bf16 memory of one or more peers at byte offset `dst_offset`.
void peer_copy_cast(const torch::Tensor& src, const std::vector<int64_t>& dst_ptrs, int64_t dst_offset_bytes) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous(), "src contiguous CUDA");
  TORCH_CHECK(dst_offset_bytes % 16 == 0, "destination offset must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(src.device());
  const long n = src.numel();
  if (n == 0) return;
  const int blocks = static_cast<int>(std::min<long>((n / 8 + 255) / 256 + 1, num_sms() * 4L));
  auto stream = at::cuda::getCurrentCUDAStream();
  for (int64_t d : dst_ptrs) {
    bf16* dst = reinterpret_cast<bf16*>(d + dst_offset_bytes);
    if (src.scalar_type() == torch::kFloat32) peer_copy_cast_kernel<float><<<blocks, 256, 0, stream>>>(src.data_ptr<float>(), dst, n);
    else if (src.scalar_type() == torch::kBFloat16)
      peer_copy_cast_kernel<bf16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(src.data_ptr()), dst, n);
    else TORCH_CHECK(false, "peer_copy_cast: src must be fp32 or bf16");
    count_launch();
  }
  TK_CUDA_CHECK(cudaGetLastError());
}

}  // namespace tk
