// Symmetric (peer-mapped) device memory for kernels that read or write other GPUs' memory over NVLink, plus the
// flag primitives they synchronise with.
//
// Allocation: plain cudaMalloc + CUDA IPC handles; the Python side exchanges the 64-byte handles through
// torch.distributed and opens every peer's buffer, which yields a table of peer base pointers for the kernels.
// Flags: 32-bit epoch counters. A producer publishes with st.release.sys after its data stores; a consumer spins with
// ld.acquire.sys for a bounded number of cycles and records PFB_ERR_WAIT_PEER in the status word when the flag never
// arrives (the process group can then be torn down from the host instead of hanging the GPU).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "sm100_common.cuh"
#include "status.h"

namespace pfb {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags[i] of every peer pad gets `value` (one thread per peer).
__global__ void peer_signal_kernel(const long long* __restrict__ peer_pads, int n_peers, int slot, int value) {
  const int i = threadIdx.x;
  if (i < n_peers) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(peer_pads[i]) + slot, value);
  }
}

// Wait until pad[slot0 + i] >= value for i < n, for at most max_ns nanoseconds of %globaltimer.
__global__ void peer_wait_kernel(const int* __restrict__ pad, int slot0, int n, int value, long long max_ns, int* status) {
  const int i = threadIdx.x;
  if (i >= n) return;
  long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  while (ld_acquire_sys(pad + slot0 + i) < value) {
    long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 > max_ns) {
      atomicCAS(status, 0, PFB_ERR_WAIT_PEER);
      return;
    }
  }
}

// dst[i] = src[i] for 16-byte vectors; src may be a peer pointer (P2P loads over NVLink).
__global__ void p2p_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n_vec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

std::tuple<int64_t, at::Tensor> symm_alloc(int64_t nbytes) {
  void* p = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&p, nbytes));
  C10_CUDA_CHECK(cudaMemset(p, 0, nbytes));
  cudaIpcMemHandle_t h;
  C10_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
  at::Tensor handle = at::empty({static_cast<int64_t>(sizeof(h))}, at::kByte);
  memcpy(handle.data_ptr(), &h, sizeof(h));
  return {reinterpret_cast<int64_t>(p), handle};
}

int64_t symm_open(const at::Tensor& handle) {
  TORCH_CHECK(handle.scalar_type() == at::kByte && handle.numel() == sizeof(cudaIpcMemHandle_t) && !handle.is_cuda());
  cudaIpcMemHandle_t h;
  memcpy(&h, handle.data_ptr(), sizeof(h));
  void* p = nullptr;
  C10_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  return reinterpret_cast<int64_t>(p);
}

void symm_close(int64_t ptr) { C10_CUDA_CHECK(cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr))); }
void symm_free(int64_t ptr) { C10_CUDA_CHECK(cudaFree(reinterpret_cast<void*>(ptr))); }

at::Tensor symm_tensor(int64_t ptr, at::IntArrayRef sizes, at::ScalarType dtype, int64_t device) {
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, device);
  return at::from_blob(reinterpret_cast<void*>(ptr), sizes, opts);
}

void peer_signal(const at::Tensor& peer_pads, int64_t slot, int64_t value) {
  TORCH_CHECK(peer_pads.is_cuda() && peer_pads.scalar_type() == at::kLong);
  const c10::cuda::CUDAGuard guard(peer_pads.device());
  peer_signal_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(reinterpret_cast<const long long*>(peer_pads.data_ptr<int64_t>()),
                                                                    static_cast<int>(peer_pads.numel()), static_cast<int>(slot),
                                                                    static_cast<int>(value));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void peer_wait(int64_t pad_ptr, int64_t slot0, int64_t n, int64_t value, double timeout_s) {
  TORCH_CHECK(n <= 32);
  const long long cycles = static_cast<long long>(timeout_s * 1e9);  // nanoseconds
  peer_wait_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(reinterpret_cast<const int*>(pad_ptr), static_cast<int>(slot0),
                                                                  static_cast<int>(n), static_cast<int>(value), cycles, status_word());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void p2p_copy(int64_t src_ptr, at::Tensor& dst, int64_t nbytes, int64_t blocks) {
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && nbytes % 16 == 0 && dst.numel() * dst.element_size() >= nbytes);
  const c10::cuda::CUDAGuard guard(dst.device());
  p2p_copy_kernel<<<static_cast<int>(blocks), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const uint4*>(src_ptr), reinterpret_cast<uint4*>(dst.data_ptr()), nbytes / 16);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("symm_alloc(int nbytes) -> (int, Tensor)", &pfb::symm_alloc);
  m.def("symm_open(Tensor handle) -> int", &pfb::symm_open);
  m.def("symm_close(int ptr) -> ()", &pfb::symm_close);
  m.def("symm_free(int ptr) -> ()", &pfb::symm_free);
  m.def("symm_tensor(int ptr, int[] sizes, ScalarType dtype, int device) -> Tensor", &pfb::symm_tensor);
  m.def("peer_signal(Tensor peer_pads, int slot, int value) -> ()", &pfb::peer_signal);
  m.def("peer_wait(int pad_ptr, int slot0, int n, int value, float timeout_s) -> ()", &pfb::peer_wait);
  m.def("p2p_copy(int src_ptr, Tensor(a!) dst, int nbytes, int blocks) -> ()", &pfb::p2p_copy);
}
