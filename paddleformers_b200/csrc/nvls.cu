// All-reduce through NVSwitch multicast memory (NVLS): every rank's buffer is bound to one multicast object, so that
//   multimem.ld_reduce  reads one address from ALL ranks and returns the sum formed inside the switch, and
//   multimem.st         writes one value to the same address on ALL ranks.
// One kernel: barrier (every rank's input is in place) -> each rank reduces its 1/tp slice with ld_reduce (fp32
// accumulation of bf16 pairs) and broadcasts the result with multimem.st -> barrier (every slice is written everywhere).
// Each GPU sends and receives 1/tp of the data per direction instead of the 2 (tp-1)/tp of a ring.
//
// The barriers are per CTA: CTA c of a rank exchanges epoch-valued flags with CTA c of every peer (flags live in the
// same symmetric allocation, written with plain peer stores, release / acquire at system scope). Every wait is bounded.
//
// Replaces the NCCL all-reduce of tensor-parallel linears without sequence parallelism
// (paddleformers/transformers/... mp_ops: _c_identity / _mp_allreduce call sites, paddleformers/nn/linear.py:39-59).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "sm100_common.cuh"
#include "status.h"

namespace pfb {

constexpr int NVLS_MAX_RANKS = 8;
constexpr int NVLS_MAX_CTAS = 64;
constexpr int NVLS_THREADS = 512;
// flag words at the start of every rank's symmetric buffer: [2 barriers][NVLS_MAX_CTAS][NVLS_MAX_RANKS]
constexpr int NVLS_FLAG_BYTES = 2 * NVLS_MAX_CTAS * NVLS_MAX_RANKS * 4;

struct NvlsPeers { int* flags[NVLS_MAX_RANKS]; };

__device__ __forceinline__ void nvls_st_release(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int nvls_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Signal CTA `cta` of every peer and wait for theirs; returns false (and records PFB_ERR_WAIT_PEER) when a peer is late.
__device__ __forceinline__ bool nvls_barrier(const NvlsPeers& peers, int which, int cta, int rank, int world, int epoch,
                                             int* status, int* s_ok) {
  const int slot = (which * NVLS_MAX_CTAS + cta) * NVLS_MAX_RANKS;
  if (static_cast<int>(threadIdx.x) < world) {
    nvls_st_release(peers.flags[threadIdx.x] + slot + rank, epoch);
    const long long t0 = global_ns(), budget = wait_budget_ns(status);
    while (nvls_ld_acquire(peers.flags[rank] + slot + threadIdx.x) < epoch) {
      if (global_ns() - t0 > budget) { atomicCAS(status, 0, PFB_ERR_WAIT_PEER); *s_ok = 0; break; }
      __nanosleep(32);
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

__global__ void __launch_bounds__(NVLS_THREADS)
nvls_allreduce_bf16_kernel(uint4* __restrict__ mc_data, long long n_vec, NvlsPeers peers, int rank, int world,
                           const int* __restrict__ epoch_ptr, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const int epoch = *epoch_ptr;
  const int cta = blockIdx.x;
  if (!nvls_barrier(peers, 0, cta, rank, world, epoch, status, &s_ok)) return;
  const long long per = (n_vec + world - 1) / world;
  const long long begin = per * rank, end = min(n_vec, begin + per);
  for (long long i = begin + static_cast<long long>(cta) * NVLS_THREADS + threadIdx.x; i < end;
       i += static_cast<long long>(gridDim.x) * NVLS_THREADS) {
    uint32_t r0, r1, r2, r3;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "l"(mc_data + i) : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_data + i), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
  }
  __threadfence_system();
  __syncthreads();
  nvls_barrier(peers, 1, cta, rank, world, epoch, status, &s_ok);
}

// mc_ptr: multicast address of the symmetric buffer; peer_ptrs: every rank's unicast address of it (int64 [world], CPU).
// The data region starts NVLS_FLAG_BYTES into the buffer and holds `numel` bf16 values (a multiple of 8).
void nvls_allreduce_bf16(int64_t mc_ptr, const at::Tensor& peer_ptrs, int64_t numel, int64_t rank, const at::Tensor& epoch) {
  TORCH_CHECK(!peer_ptrs.is_cuda() && peer_ptrs.scalar_type() == at::kLong && peer_ptrs.numel() <= NVLS_MAX_RANKS);
  TORCH_CHECK(epoch.is_cuda() && epoch.scalar_type() == at::kInt && numel % 8 == 0 && mc_ptr != 0);
  const c10::cuda::CUDAGuard guard(epoch.device());
  const int world = static_cast<int>(peer_ptrs.numel());
  NvlsPeers peers{};
  for (int q = 0; q < world; ++q) peers.flags[q] = reinterpret_cast<int*>(peer_ptrs.data_ptr<int64_t>()[q]);
  const long long n_vec = numel / 8;
  const long long per = (n_vec + world - 1) / world;
  const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(NVLS_MAX_CTAS, (per + NVLS_THREADS - 1) / NVLS_THREADS)));
  nvls_allreduce_bf16_kernel<<<grid, NVLS_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<uint4*>(mc_ptr + NVLS_FLAG_BYTES), n_vec, peers, static_cast<int>(rank), world, epoch.data_ptr<int>(),
      status_word());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

int64_t nvls_flag_bytes() { return NVLS_FLAG_BYTES; }

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("nvls_allreduce_bf16(int mc_ptr, Tensor peer_ptrs, int numel, int rank, Tensor epoch) -> ()", &pfb::nvls_allreduce_bf16);
  m.def("nvls_flag_bytes() -> int", &pfb::nvls_flag_bytes);
}
