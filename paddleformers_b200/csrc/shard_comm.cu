// Optimizer-sharding collectives fused with the arithmetic around them, over NVLink peer memory (sm_100a).
//
//   shard_reduce   this rank's slice of the flat fp32 gradient = scale * sum over the sharding ranks of their copies of
//                  that slice, read straight out of the peers' gradient buffers (plain 16-byte peer loads, fixed rank
//                  order: deterministic), written over the local copy, with the slice's squared norm accumulated on the
//                  way. Replaces reduce-scatter + scale + norm pass (three passes over the slice) by one.
//   adamw_push     the AdamW update of the slice (fp32 master weights and moments) whose bf16 result is stored into
//                  EVERY rank's flat parameter buffer: the parameter all-gather is the update's own output and needs no
//                  second pass and no staging copy.
//
// Ordering between ranks uses epoch flags in symmetric memory (shard_signal / the waits inside the kernels):
//   "grads final"   raised by a rank after its last backward kernel; shard_reduce waits for it from every rank before
//                   reading, which also tells it that nobody still reads the old parameters (adamw_push may then write);
//   "params pushed" raised after adamw_push; every rank waits for it from all ranks before it zeroes its gradient buffer
//                   (peers have finished reading it) and before its next forward pass reads the parameters.
// Every wait is bounded and reports PFB_ERR_WAIT_PEER. The reference overlaps the same two collectives with compute
// (paddleformers/trainer/training_args.py:1593-1640, trainer/trainer.py:2692-2696, :4326-4332); its reduce-scatter,
// optimizer and all-gather are three library calls with their own passes over memory.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "gemm_comm_sm100.cuh"
#include "status.h"

namespace pfb {

constexpr int SH_MAX_RANKS = 8;
struct ShardPeers {
  const float* grad[SH_MAX_RANKS];     // every rank's flat fp32 gradient buffer
  __nv_bfloat16* param[SH_MAX_RANKS];  // every rank's flat bf16 parameter buffer
  int* flags[SH_MAX_RANKS];            // every rank's flag pad: [2][SH_MAX_RANKS] (kind, source rank)
};

// flags[kind][rank] = epoch on every peer (stream-ordered after this rank's earlier work)
__global__ void shard_signal_kernel(ShardPeers peers, int n, int rank, int kind, const int* __restrict__ epoch_ptr) {
  const int q = threadIdx.x;
  if (q >= n) return;
  __threadfence_system();
  st_release_sys_i32(peers.flags[q] + kind * SH_MAX_RANKS + rank, *epoch_ptr);
}

// Bounded wait of one CTA for flags[kind][0..n) >= epoch; returns false (and records the status) on time-out.
__device__ __forceinline__ bool shard_wait_all(const int* flags, int kind, int n, int epoch, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < n) {
    const long long t0 = global_ns(), budget = wait_budget_ns(status);
    while (ld_acquire_sys_i32(flags + kind * SH_MAX_RANKS + threadIdx.x) < epoch) {
      if (global_ns() - t0 > budget) { atomicCAS(status, 0, PFB_ERR_WAIT_PEER); s_ok = 0; break; }
      __nanosleep(128);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void shard_wait_kernel(const int* __restrict__ flags, int kind, int n, const int* __restrict__ epoch_ptr, int* status) {
  shard_wait_all(flags, kind, n, *epoch_ptr, status);
}

// Sum of a value over the block in a fixed order (warp butterflies, then the warp sums): the same tree as the squared
// norm kernel of the unfused path, so that both paths give the same bits for the same slice.
__device__ __forceinline__ float shard_block_sum(float v, float* red) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = l < nw ? red[l] : 0.f;
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

// norm_acc[0] += sum of the per-block partials, in index order
__global__ void shard_norm_finish_kernel(const float* __restrict__ partial, int P, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += partial[i];
  s = shard_block_sum(s, red);
  if (threadIdx.x == 0) out[0] += s;
}

// out slice (local gradient buffer, elements [lo, lo + cnt)) = scale * sum_q grad_q[lo + i]; partial[blockIdx.x] = this
// block's share of the slice's squared norm (no atomics: the sum is the same on every run).
__global__ void __launch_bounds__(256) shard_reduce_kernel(ShardPeers peers, int n, int rank, long long lo, long long cnt, float scale,
                                                           float* __restrict__ out, float* __restrict__ partial,
                                                           const int* __restrict__ epoch_ptr, int* status) {
  if (!shard_wait_all(peers.flags[rank], 0, n, *epoch_ptr, status)) { if (threadIdx.x == 0) partial[blockIdx.x] = 0.f; return; }
  const long long nv = cnt >> 2;
  float sq = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    #pragma unroll
    for (int q = 0; q < SH_MAX_RANKS; ++q) {
      if (q < n) {
        const float4 v = reinterpret_cast<const float4*>(peers.grad[q] + lo)[i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(out + lo)[i] = acc;
    sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  __shared__ float red[32];
  sq = shard_block_sum(sq, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = sq;
}

// AdamW on the slice; the bf16 weights go to elements [lo, lo + cnt) of every rank's parameter buffer.
// scalars: [0] lr, [1] gradient multiplier, [2] 1 - beta1^t, [3] 1 - beta2^t, [4] skip flag.
__global__ void __launch_bounds__(256) adamw_push_kernel(ShardPeers peers, int n, int rank, long long lo, long long cnt,
                                                         float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                                         const float* __restrict__ g, const float* __restrict__ scalars, float beta1,
                                                         float beta2, float eps, float wd) {
  const bool skip = scalars[4] != 0.f;       // non-finite gradient: weights stay as they are (and equal on every rank)
  if (skip) return;
  const float lr = scalars[0], gmul = scalars[1], bc1 = scalars[2], bc2 = scalars[3];
  const long long nv = cnt >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i], mm = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
    const float4 gg = reinterpret_cast<const float4*>(g + lo)[i];
    float* P = reinterpret_cast<float*>(&pp); float* Mm = reinterpret_cast<float*>(&mm); float* Vv = reinterpret_cast<float*>(&vv);
    const float* G = reinterpret_cast<const float*>(&gg);
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = G[j] * gmul;
      Mm[j] = beta1 * Mm[j] + (1.f - beta1) * gr;
      Vv[j] = beta2 * Vv[j] + (1.f - beta2) * gr * gr;
      P[j] = P[j] * (1.f - lr * wd) - lr * (Mm[j] / bc1) / (sqrtf(Vv[j] / bc2) + eps);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    uint2 o;
    o.x = pack_bf16x2(P[0], P[1]);
    o.y = pack_bf16x2(P[2], P[3]);
    #pragma unroll
    for (int q = 0; q < SH_MAX_RANKS; ++q)
      if (q < n) reinterpret_cast<uint2*>(peers.param[(rank + q) % n] + lo)[i] = o;     // own copy first, then round the ring
  }
}

static ShardPeers make_shard_peers(const at::Tensor& grad_ptrs, const at::Tensor& param_ptrs, const at::Tensor& flag_ptrs, int n) {
  TORCH_CHECK(n >= 1 && n <= SH_MAX_RANKS && !grad_ptrs.is_cuda() && grad_ptrs.scalar_type() == at::kLong);
  TORCH_CHECK(grad_ptrs.numel() == n && param_ptrs.numel() == n && flag_ptrs.numel() == n);
  ShardPeers sp{};
  for (int q = 0; q < n; ++q) {
    sp.grad[q] = reinterpret_cast<const float*>(grad_ptrs.data_ptr<int64_t>()[q]);
    sp.param[q] = reinterpret_cast<__nv_bfloat16*>(param_ptrs.data_ptr<int64_t>()[q]);
    sp.flags[q] = reinterpret_cast<int*>(flag_ptrs.data_ptr<int64_t>()[q]);
  }
  return sp;
}

// the grid of the squared-norm kernel of the unfused path (same partition of the slice -> same partial sums)
static int shard_grid(long long cnt) {
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return static_cast<int>(std::max<long long>(1, std::min<long long>((cnt / 4 + 255) / 256 + 1, static_cast<long long>(sms) * 8)));
}

void shard_signal(const at::Tensor& grad_ptrs, const at::Tensor& param_ptrs, const at::Tensor& flag_ptrs, int64_t rank, int64_t kind,
                  const at::Tensor& epoch) {
  const int n = grad_ptrs.numel();
  shard_signal_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(make_shard_peers(grad_ptrs, param_ptrs, flag_ptrs, n), n,
                                                                     static_cast<int>(rank), static_cast<int>(kind), epoch.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void shard_wait(const at::Tensor& flag_ptrs, int64_t rank, int64_t kind, const at::Tensor& epoch) {
  const int n = flag_ptrs.numel();
  const int* flags = reinterpret_cast<const int*>(flag_ptrs.data_ptr<int64_t>()[rank]);
  shard_wait_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(flags, static_cast<int>(kind), n, epoch.data_ptr<int>(), status_word());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

// local_grad: this rank's flat fp32 gradient buffer; elements [lo, lo + cnt) become the reduced, scaled slice.
void shard_reduce(at::Tensor& local_grad, const at::Tensor& grad_ptrs, const at::Tensor& param_ptrs, const at::Tensor& flag_ptrs,
                  int64_t rank, int64_t lo, int64_t cnt, double scale, at::Tensor& norm_acc, const at::Tensor& epoch) {
  TORCH_CHECK(local_grad.is_cuda() && local_grad.scalar_type() == at::kFloat && local_grad.is_contiguous());
  TORCH_CHECK(lo % 4 == 0 && cnt % 4 == 0 && lo + cnt <= local_grad.numel(), "shard_reduce: slice must be 16-byte aligned");
  TORCH_CHECK(norm_acc.scalar_type() == at::kFloat && norm_acc.numel() >= 1);
  const c10::cuda::CUDAGuard guard(local_grad.device());
  const int n = grad_ptrs.numel();
  const int P = shard_grid(cnt);
  at::Tensor partial = at::empty({P}, norm_acc.options());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  shard_reduce_kernel<<<P, 256, 0, stream>>>(
      make_shard_peers(grad_ptrs, param_ptrs, flag_ptrs, n), n, static_cast<int>(rank), lo, cnt, static_cast<float>(scale),
      local_grad.data_ptr<float>(), partial.data_ptr<float>(), epoch.data_ptr<int>(), status_word());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  shard_norm_finish_kernel<<<1, 256, 0, stream>>>(partial.data_ptr<float>(), P, norm_acc.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
}

void adamw_push(at::Tensor& master, at::Tensor& m, at::Tensor& v, const at::Tensor& local_grad, const at::Tensor& grad_ptrs,
                const at::Tensor& param_ptrs, const at::Tensor& flag_ptrs, int64_t rank, int64_t lo, const at::Tensor& scalars,
                double beta1, double beta2, double eps, double wd) {
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  const long long cnt = master.numel();
  TORCH_CHECK(m.numel() == cnt && v.numel() == cnt && lo % 4 == 0 && cnt % 4 == 0 && lo + cnt <= local_grad.numel());
  const c10::cuda::CUDAGuard guard(master.device());
  const int n = grad_ptrs.numel();
  adamw_push_kernel<<<shard_grid(cnt), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      make_shard_peers(grad_ptrs, param_ptrs, flag_ptrs, n), n, static_cast<int>(rank), lo, cnt, master.data_ptr<float>(),
      m.data_ptr<float>(), v.data_ptr<float>(), local_grad.data_ptr<float>(), scalars.data_ptr<float>(), static_cast<float>(beta1),
      static_cast<float>(beta2), static_cast<float>(eps), static_cast<float>(wd));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("shard_signal(Tensor grad_ptrs, Tensor param_ptrs, Tensor flag_ptrs, int rank, int kind, Tensor epoch) -> ()", &pfb::shard_signal);
  m.def("shard_wait(Tensor flag_ptrs, int rank, int kind, Tensor epoch) -> ()", &pfb::shard_wait);
  m.def("shard_reduce(Tensor(a!) local_grad, Tensor grad_ptrs, Tensor param_ptrs, Tensor flag_ptrs, int rank, int lo, int cnt, "
        "float scale, Tensor(b!) norm_acc, Tensor epoch) -> ()", &pfb::shard_reduce);
  m.def("adamw_push(Tensor(a!) master, Tensor(b!) m, Tensor(c!) v, Tensor local_grad, Tensor grad_ptrs, Tensor param_ptrs, "
        "Tensor flag_ptrs, int rank, int lo, Tensor scalars, float beta1, float beta2, float eps, float wd) -> ()", &pfb::adamw_push);
}
