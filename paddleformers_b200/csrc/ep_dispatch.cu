// Expert-parallel token dispatch / combine over NVLink peer memory, without NCCL and without host synchronisation.
//
// Three kernels replace the all-to-all exchange of an MoE layer (the role DeepEP plays for the reference,
// paddleformers/transformers/fused_a2a.py:81-178, whose dispatch waits on the host for the receive counts):
//
//   ep_exchange   one CTA per GPU. Pushes this rank's per-expert pair counts to every destination rank, waits
//                 (bounded) for everybody's counts, lays the local receive buffer out as expert-sorted segments
//                 padded to 128 rows (block -> expert table for the grouped GEMM), and pushes to every source rank
//                 the slot at which that source's rows of each local expert start.
//   ep_push_rows  one warp per routed (token, expert) pair: copies the token's row (optionally scaled by a per-pair
//                 factor) into its slot of the destination's receive buffer with 16-byte peer stores. The last CTA to
//                 finish raises a "rows delivered" flag on every peer.
//   ep_pull_rows  one warp per token: reads the k rows that belong to the token from the peers' buffers with 16-byte
//                 peer loads and writes their (optionally weighted) sum - the combine, and the backward of dispatch.
//                 Optionally also returns the k dot products <row, g[token]> (gradient of the routing weights).
//
// All flags are epoch-valued; all waits are bounded and report PFB_ERR_WAIT_PEER. A pair whose slot lies beyond the
// receive capacity is DROPPED (capacity-factor semantics: it is not sent and contributes nothing to the combine, forward
// and backward) and counted in the second word of the status block, which the host reads with read_drop_count.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "gemm_comm_sm100.cuh"
#include "status.h"

namespace pfb {

constexpr int EP_MAX_RANKS = 8;
constexpr int EP_MAX_LOCAL_EXPERTS = 128;

struct EpTables {
  // symmetric int32 region per rank (see layout in fused_ep.py):
  int* peer_base[EP_MAX_RANKS];
  int* base;
};

// table layout (ints): [0, ep*EL) counts[src][e] | [ep*EL, 2*ep*EL) offsets[dst][e] (written by dst for me)
//                      | flags: A[ep], B[ep], C[ep], D[ep] | misc
__device__ __forceinline__ int tab_counts(int ep, int EL) { return 0; }
__device__ __forceinline__ int tab_offsets(int ep, int EL) { return ep * EL; }
__device__ __forceinline__ int tab_flags(int ep, int EL) { return 2 * ep * EL; }

__global__ void ep_exchange_kernel(EpTables tabs, const int* __restrict__ my_counts /*[ep*EL]*/, int* __restrict__ block_expert,
                                   int n_blocks, int* __restrict__ expert_rows /*[EL,2]*/, int* __restrict__ total_rows,
                                   int* __restrict__ expert_tot /*[EL] rows received per expert before padding, or null*/,
                                   int rank, int ep, int EL, const int* __restrict__ epoch_ptr, int* status) {
  __shared__ int s_cnt[EP_MAX_RANKS * EP_MAX_LOCAL_EXPERTS];
  __shared__ int s_seg[EP_MAX_LOCAL_EXPERTS + 1];
  __shared__ int s_ok;
  const int epoch = *epoch_ptr;
  const int tid = threadIdx.x;
  const int FL = tab_flags(ep, EL);
  if (tid == 0) s_ok = 1;
  // phase A: my counts for destination d go to d's table row [rank]
  for (int i = tid; i < ep * EL; i += blockDim.x) {
    const int d = i / EL, e = i - d * EL;
    tabs.peer_base[d][tab_counts(ep, EL) + rank * EL + e] = my_counts[i];
  }
  __threadfence_system();
  __syncthreads();
  if (tid < ep) st_release_sys_i32(tabs.peer_base[tid] + FL + 0 * EP_MAX_RANKS + rank, epoch);
  // phase B: wait for all sources' counts
  if (tid < ep) {
    const long long t0 = global_ns(), budget = wait_budget_ns(status);
    while (ld_acquire_sys_i32(tabs.base + FL + 0 * EP_MAX_RANKS + tid) < epoch) {
      if (global_ns() - t0 > budget) { atomicCAS(status, 0, PFB_ERR_WAIT_PEER); s_ok = 0; break; }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (!s_ok) return;
  for (int i = tid; i < ep * EL; i += blockDim.x) s_cnt[i] = *(reinterpret_cast<volatile int*>(tabs.base) + tab_counts(ep, EL) + i);
  __syncthreads();
  if (tid == 0) {
    int pos = 0;
    for (int e = 0; e < EL; ++e) {
      int tot = 0;
      for (int s = 0; s < ep; ++s) tot += s_cnt[s * EL + e];
      s_seg[e] = pos;
      int padded = (tot + 127) / 128 * 128;
      // receive buffer too small: clamp so that no consumer leaves the buffer; the senders drop (and count) the pairs
      // whose slot falls beyond it
      if (pos + padded > n_blocks * 128) padded = max(0, n_blocks * 128 - pos);
      expert_rows[2 * e] = pos;
      expert_rows[2 * e + 1] = padded;
      if (expert_tot) expert_tot[e] = min(tot, padded);
      pos += padded;
    }
    s_seg[EL] = pos;
    total_rows[0] = pos;
  }
  __syncthreads();
  // block -> expert table
  for (int b = tid; b < n_blocks; b += blockDim.x) {
    const int r = b * 128;
    int e = -1;
    if (r < s_seg[EL]) {
      e = 0;
      while (e + 1 < EL && s_seg[e + 1] <= r) ++e;
      // skip empty experts (their segment has zero rows, so s_seg[e + 1] == s_seg[e])
    }
    block_expert[b] = e;
  }
  // phase C: tell each source where its rows of each of my experts start
  for (int i = tid; i < ep * EL; i += blockDim.x) {
    const int s = i / EL, e = i - s * EL;
    int off = s_seg[e];
    for (int q = 0; q < s; ++q) off += s_cnt[q * EL + e];
    tabs.peer_base[s][tab_offsets(ep, EL) + rank * EL + e] = off;
  }
  __threadfence_system();
  __syncthreads();
  if (tid < ep) st_release_sys_i32(tabs.peer_base[tid] + FL + 1 * EP_MAX_RANKS + rank, epoch);
  // phase D: wait for the offsets from every destination
  if (tid < ep) {
    const long long t0 = global_ns(), budget = wait_budget_ns(status);
    while (ld_acquire_sys_i32(tabs.base + FL + 1 * EP_MAX_RANKS + tid) < epoch) {
      if (global_ns() - t0 > budget) { atomicCAS(status, 0, PFB_ERR_WAIT_PEER); break; }
      __nanosleep(64);
    }
  }
}

struct EpPeers { __nv_bfloat16* buf[EP_MAX_RANKS]; int* flag_base[EP_MAX_RANKS]; };

// pair p = (token p / k, slot j = p % k): destination rank and slot from the offsets table.
__global__ void ep_push_rows_kernel(const __nv_bfloat16* __restrict__ x, const long long* __restrict__ idx /*[T*k] global expert*/,
                                    const int* __restrict__ rank_in_expert /*[T*k]*/, const float* __restrict__ scale /*[T*k] or null*/,
                                    const int* __restrict__ offsets /*[ep*EL]*/, int* __restrict__ pair_slot /*[T*k] out*/,
                                    EpPeers peers, int n_pairs, int k, int H, int EL, int ep, int capacity_rows, int rank,
                                    int flag_slot, const int* __restrict__ epoch_ptr, int* __restrict__ done_counter, int* status) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int nv = H >> 3;
  for (int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < n_pairs; p += warps) {
    const long long e = idx[p];
    const int d = static_cast<int>(e / EL), el = static_cast<int>(e - static_cast<long long>(d) * EL);
    // forward: the slot comes from the offsets table of this exchange and is recorded; backward (offsets == nullptr):
    // the recorded slot is reused, because the table already belongs to a later exchange
    const int slot = offsets ? offsets[d * EL + el] + rank_in_expert[p] : pair_slot[p];
    if (offsets && lane == 0) pair_slot[p] = slot;
    if (slot >= capacity_rows) {   // dropped pair: nothing is sent, the combine adds nothing for it; counted once, in the forward pass
      if (lane == 0 && offsets) atomicAdd(status + 1, 1);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(p / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(peers.buf[d] + static_cast<long long>(slot) * H);
    if (scale == nullptr) {
      for (int i = lane; i < nv; i += 32) dst[i] = src[i];
    } else {
      const float sc = scale[p];
      for (int i = lane; i < nv; i += 32) {
        uint4 v = src[i];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          h[j] = __float22bfloat162_rn(make_float2(f.x * sc, f.y * sc));
        }
        dst[i] = v;
      }
    }
  }
  // the last CTA to finish tells every peer that this rank's rows have been delivered
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(done_counter, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      *done_counter = 0;
      __threadfence_system();
      const int epoch = *epoch_ptr;
      for (int q = 0; q < ep; ++q) st_release_sys_i32(peers.flag_base[q] + flag_slot * EP_MAX_RANKS + rank, epoch);
    }
  }
}

// out[t] = sum_j w[t, j] * peer_buf[dest(t, j)][slot(t, j)]  (w == nullptr: plain sum); optional dots[t, j] = <row, g[t]>
__global__ void ep_pull_rows_kernel(__nv_bfloat16* __restrict__ out, const long long* __restrict__ idx, const int* __restrict__ pair_slot,
                                    const float* __restrict__ w, const __nv_bfloat16* __restrict__ g, float* __restrict__ dots,
                                    EpPeers peers, int T, int k, int H, int EL, int capacity_rows) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int nv = H >> 3;  // H <= 8192: up to 32 vectors per lane is too many registers, so loop over 256-element chunks
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    for (int i0 = 0; i0 < nv; i0 += 32) {
      const int i = i0 + lane;
      float acc[8];
      #pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      float gv[8];
      #pragma unroll
      for (int j = 0; j < 8; ++j) gv[j] = 0.f;
      if (g != nullptr && i < nv) {
        const uint4 graw = reinterpret_cast<const uint4*>(g + static_cast<long long>(t) * H)[i];
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
        #pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(gh[j]); gv[2 * j] = f.x; gv[2 * j + 1] = f.y; }
      }
      for (int j0 = 0; j0 < k; j0 += 4) {
        uint4 v[4];
        float wj[4];
        bool have[4];
        #pragma unroll
        for (int u = 0; u < 4; ++u) {   // issue the (up to) four peer loads before using any of them
          const int j = j0 + u;
          have[u] = false;
          wj[u] = 0.f;
          v[u] = make_uint4(0u, 0u, 0u, 0u);
          if (j < k) {
            const int p = t * k + j;
            const int slot = pair_slot[p];
            if (slot < capacity_rows && i < nv) {
              const int d = static_cast<int>(idx[p] / EL);
              v[u] = reinterpret_cast<const uint4*>(peers.buf[d] + static_cast<long long>(slot) * H)[i];
              wj[u] = w ? w[p] : 1.f;
              have[u] = true;
            }
          }
        }
        #pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = j0 + u;
          if (j >= k) break;
          float dot = 0.f;
          if (have[u]) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
            #pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = __bfloat1622float2(h[q]);
              acc[2 * q] += wj[u] * f.x; acc[2 * q + 1] += wj[u] * f.y;
              dot += f.x * gv[2 * q] + f.y * gv[2 * q + 1];
            }
          }
          if (dots != nullptr) {
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (lane == 0) {
              const int p = t * k + j;
              if (i0 == 0) dots[p] = dot; else dots[p] += dot;
            }
          }
        }
      }
      if (out != nullptr && i < nv) {
        reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H)[i] = make_uint4(
            pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
static EpTables make_tabs(const at::Tensor& peer_tab_ptrs, int rank, int ep) {
  EpTables t{};
  for (int q = 0; q < ep; ++q) t.peer_base[q] = reinterpret_cast<int*>(peer_tab_ptrs.data_ptr<int64_t>()[q]);
  t.base = t.peer_base[rank];
  return t;
}
static EpPeers make_peers(const at::Tensor& peer_buf_ptrs, const at::Tensor& peer_tab_ptrs, int ep, int EL) {
  EpPeers p{};
  for (int q = 0; q < ep; ++q) {
    p.buf[q] = reinterpret_cast<__nv_bfloat16*>(peer_buf_ptrs.data_ptr<int64_t>()[q]);
    p.flag_base[q] = reinterpret_cast<int*>(peer_tab_ptrs.data_ptr<int64_t>()[q]) + 2 * ep * EL;
  }
  return p;
}

void ep_exchange(const at::Tensor& peer_tab_ptrs, const at::Tensor& my_counts, at::Tensor& block_expert, at::Tensor& expert_rows,
                 at::Tensor& total_rows, int64_t rank, int64_t ep, int64_t EL, const at::Tensor& epoch,
                 c10::optional<at::Tensor> expert_tot) {
  TORCH_CHECK(ep <= EP_MAX_RANKS && EL <= EP_MAX_LOCAL_EXPERTS && my_counts.scalar_type() == at::kInt && my_counts.numel() == ep * EL);
  TORCH_CHECK(block_expert.scalar_type() == at::kInt && expert_rows.scalar_type() == at::kInt && expert_rows.numel() == 2 * EL);
  const c10::cuda::CUDAGuard guard(my_counts.device());
  ep_exchange_kernel<<<1, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      make_tabs(peer_tab_ptrs, rank, ep), my_counts.data_ptr<int>(), block_expert.data_ptr<int>(), static_cast<int>(block_expert.numel()),
      expert_rows.data_ptr<int>(), total_rows.data_ptr<int>(), expert_tot.has_value() ? expert_tot->data_ptr<int>() : nullptr, rank, ep, EL,
      epoch.data_ptr<int>(), status_word());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void ep_push_rows(const at::Tensor& x, const at::Tensor& idx, const at::Tensor& rank_in_expert, const c10::optional<at::Tensor>& scale,
                  const at::Tensor& peer_tab_ptrs, at::Tensor& pair_slot, const at::Tensor& peer_buf_ptrs, int64_t k, int64_t EL,
                  int64_t ep, int64_t capacity_rows, int64_t rank, int64_t flag_slot, const at::Tensor& epoch, at::Tensor& done_counter,
                  bool slots_from_table) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16 && x.size(1) % 8 == 0);
  TORCH_CHECK(idx.scalar_type() == at::kLong && idx.is_contiguous() && rank_in_expert.scalar_type() == at::kInt);
  const c10::cuda::CUDAGuard guard(x.device());
  const int n_pairs = idx.numel(), H = x.size(1);
  TORCH_CHECK(x.size(0) * k == n_pairs);
  int* tab = reinterpret_cast<int*>(peer_tab_ptrs.data_ptr<int64_t>()[rank]);
  const int blocks = std::max(1, std::min((n_pairs * 32 + 255) / 256, at::cuda::getCurrentDeviceProperties()->multiProcessorCount * 8));
  ep_push_rows_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()),
      rank_in_expert.data_ptr<int>(), scale.has_value() ? scale->data_ptr<float>() : nullptr, slots_from_table ? tab + ep * EL : nullptr,
      pair_slot.data_ptr<int>(),
      make_peers(peer_buf_ptrs, peer_tab_ptrs, ep, EL), n_pairs, k, H, EL, ep, capacity_rows, rank, flag_slot, epoch.data_ptr<int>(),
      done_counter.data_ptr<int>(), status_word());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void ep_wait_flag(const at::Tensor& peer_tab_ptrs, int64_t rank, int64_t ep, int64_t EL, int64_t flag_slot, const at::Tensor& epoch);

__global__ void ep_wait_flag_kernel(const int* __restrict__ flags, int ep, const int* __restrict__ epoch_ptr, int* status) {
  const int tid = threadIdx.x;
  if (tid >= ep) return;
  const int epoch = *epoch_ptr;
  const long long t0 = global_ns(), budget = wait_budget_ns(status);
  while (ld_acquire_sys_i32(flags + tid) < epoch) {
    if (global_ns() - t0 > budget) { atomicCAS(status, 0, PFB_ERR_WAIT_PEER); return; }
    __nanosleep(64);
  }
}

void ep_wait_flag(const at::Tensor& peer_tab_ptrs, int64_t rank, int64_t ep, int64_t EL, int64_t flag_slot, const at::Tensor& epoch) {
  int* tab = reinterpret_cast<int*>(peer_tab_ptrs.data_ptr<int64_t>()[rank]);
  ep_wait_flag_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(tab + 2 * ep * EL + flag_slot * EP_MAX_RANKS, ep,
                                                                     epoch.data_ptr<int>(), status_word());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

__global__ void ep_signal_flag_kernel(EpPeers peers, int ep, int rank, int flag_slot, const int* __restrict__ epoch_ptr) {
  const int tid = threadIdx.x;
  if (tid >= ep) return;
  __threadfence_system();
  st_release_sys_i32(peers.flag_base[tid] + flag_slot * EP_MAX_RANKS + rank, *epoch_ptr);
}

void ep_signal_flag(const at::Tensor& peer_tab_ptrs, int64_t rank, int64_t ep, int64_t EL, int64_t flag_slot, const at::Tensor& epoch) {
  ep_signal_flag_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(make_peers(peer_tab_ptrs, peer_tab_ptrs, ep, EL), ep, rank,
                                                                       flag_slot, epoch.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void ep_pull_rows(c10::optional<at::Tensor> out, const at::Tensor& idx, const at::Tensor& pair_slot, const c10::optional<at::Tensor>& w,
                  const c10::optional<at::Tensor>& g, c10::optional<at::Tensor> dots, const at::Tensor& peer_buf_ptrs,
                  const at::Tensor& peer_tab_ptrs, int64_t T, int64_t k, int64_t H, int64_t EL, int64_t ep, int64_t capacity_rows) {
  const c10::cuda::CUDAGuard guard(idx.device());
  TORCH_CHECK(H % 8 == 0 && idx.numel() == T * k);
  const int blocks = std::max<int64_t>(1, std::min<int64_t>((T * 32 + 255) / 256, at::cuda::getCurrentDeviceProperties()->multiProcessorCount * 8));
  ep_pull_rows_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      out.has_value() ? reinterpret_cast<__nv_bfloat16*>(out->data_ptr()) : nullptr, reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()),
      pair_slot.data_ptr<int>(), w.has_value() ? w->data_ptr<float>() : nullptr,
      g.has_value() ? reinterpret_cast<const __nv_bfloat16*>(g->data_ptr()) : nullptr, dots.has_value() ? dots->data_ptr<float>() : nullptr,
      make_peers(peer_buf_ptrs, peer_tab_ptrs, ep, EL), T, k, H, EL, capacity_rows);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

// ---- routing-weight gradient formed on the expert's side -----------------------------------------------------------
// rowdots[slot] = <y[slot, :], dy[slot, :]> for the rows this rank's experts hold (one warp per row). dy rows are w * dout,
// so the source rank recovers <y_row, dout> = rowdots / w and never re-reads the expert outputs across NVLink.
__global__ void ep_row_dots_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dy, float* __restrict__ rowdots,
                                   const int* __restrict__ expert_rows, int EL, int H, int capacity_rows) {
  const int lane = threadIdx.x & 31;
  const int rows = min(capacity_rows, expert_rows[2 * (EL - 1)] + expert_rows[2 * (EL - 1) + 1]);
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int nv = H >> 3;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const uint4* a = reinterpret_cast<const uint4*>(y + static_cast<long long>(r) * H);
    const uint4* b = reinterpret_cast<const uint4*>(dy + static_cast<long long>(r) * H);
    float acc = 0.f;
    for (int i = lane; i < nv; i += 32) {
      const uint4 va = a[i], vb = b[i];
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&va);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&vb);
      #pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 fa = __bfloat1622float2(ha[q]), fb = __bfloat1622float2(hb[q]);
        acc += fa.x * fb.x + fa.y * fb.y;
      }
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) rowdots[r] = acc;
  }
}

// Zero the padding rows of every expert segment (rows [start + received, start + padded)): the weight-gradient GEMMs read
// whole 128-row blocks. One warp per row, 16-byte stores. Peers only ever write the received rows, so this may run while
// their pushes for the same exchange arrive.
__global__ void ep_zero_padding_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ expert_rows, const int* __restrict__ expert_tot,
                                       int EL, int H, int capacity_rows) {
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = (gridDim.x * blockDim.x) >> 5;
  const int nv = H >> 3;
  for (int w = warp; w < EL * 128; w += warps) {
    const int e = w >> 7, r = w & 127;
    const int start = expert_rows[2 * e], padded = expert_rows[2 * e + 1], tot = expert_tot[e];
    const int row = start + tot + r;
    if (tot + r >= padded || row >= capacity_rows) continue;
    uint4* dst = reinterpret_cast<uint4*>(buf + static_cast<long long>(row) * H);
    for (int i = lane; i < nv; i += 32) dst[i] = make_uint4(0u, 0u, 0u, 0u);
  }
}

void ep_zero_padding(at::Tensor& buf, const at::Tensor& expert_rows, const at::Tensor& expert_tot, int64_t EL) {
  TORCH_CHECK(buf.is_cuda() && buf.scalar_type() == at::kBFloat16 && buf.is_contiguous() && buf.size(1) % 8 == 0);
  TORCH_CHECK(expert_rows.scalar_type() == at::kInt && expert_rows.numel() == 2 * EL && expert_tot.scalar_type() == at::kInt &&
              expert_tot.numel() == EL);
  const c10::cuda::CUDAGuard guard(buf.device());
  const int blocks = static_cast<int>((EL * 128 * 32 + 255) / 256);
  ep_zero_padding_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<__nv_bfloat16*>(buf.data_ptr()), expert_rows.data_ptr<int>(), expert_tot.data_ptr<int>(), static_cast<int>(EL),
      static_cast<int>(buf.size(1)), static_cast<int>(buf.size(0)));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

struct EpScalarPeers { const float* buf[EP_MAX_RANKS]; };

// dots[p] = rowdots_of_destination[slot(p)] / w[p] (0 for dropped pairs and for w == 0): 4 bytes per pair across NVLink
__global__ void ep_pull_scalars_kernel(float* __restrict__ dots, const long long* __restrict__ idx, const int* __restrict__ pair_slot,
                                       const float* __restrict__ w, EpScalarPeers peers, int n_pairs, int EL, int capacity_rows) {
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += gridDim.x * blockDim.x) {
    const int slot = pair_slot[p];
    const float wp = w[p];
    float v = 0.f;
    if (slot < capacity_rows && wp != 0.f) v = peers.buf[static_cast<int>(idx[p] / EL)][slot] / wp;
    dots[p] = v;
  }
}

void ep_row_dots(const at::Tensor& y, const at::Tensor& dy, at::Tensor& rowdots, const at::Tensor& expert_rows, int64_t EL) {
  TORCH_CHECK(y.is_cuda() && y.scalar_type() == at::kBFloat16 && dy.scalar_type() == at::kBFloat16 && y.is_contiguous() && dy.is_contiguous());
  TORCH_CHECK(y.sizes() == dy.sizes() && y.size(1) % 8 == 0 && rowdots.scalar_type() == at::kFloat && rowdots.numel() >= y.size(0));
  TORCH_CHECK(expert_rows.scalar_type() == at::kInt && expert_rows.numel() == 2 * EL);
  const c10::cuda::CUDAGuard guard(y.device());
  const int blocks = at::cuda::getCurrentDeviceProperties()->multiProcessorCount * 8;
  ep_row_dots_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(y.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()), rowdots.data_ptr<float>(),
      expert_rows.data_ptr<int>(), static_cast<int>(EL), static_cast<int>(y.size(1)), static_cast<int>(y.size(0)));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void ep_pull_scalars(at::Tensor& dots, const at::Tensor& idx, const at::Tensor& pair_slot, const at::Tensor& w,
                     const at::Tensor& peer_rowdots_ptrs, int64_t EL, int64_t ep, int64_t capacity_rows) {
  TORCH_CHECK(dots.is_cuda() && dots.scalar_type() == at::kFloat && w.scalar_type() == at::kFloat && dots.numel() == idx.numel() &&
              w.numel() == idx.numel() && ep <= EP_MAX_RANKS && !peer_rowdots_ptrs.is_cuda());
  const c10::cuda::CUDAGuard guard(dots.device());
  EpScalarPeers peers{};
  for (int q = 0; q < ep; ++q) peers.buf[q] = reinterpret_cast<const float*>(peer_rowdots_ptrs.data_ptr<int64_t>()[q]);
  const int n = static_cast<int>(idx.numel());
  if (n == 0) return;
  ep_pull_scalars_kernel<<<std::min((n + 255) / 256, 148 * 8), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      dots.data_ptr<float>(), reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), pair_slot.data_ptr<int>(), w.data_ptr<float>(),
      peers, n, static_cast<int>(EL), static_cast<int>(capacity_rows));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("ep_row_dots(Tensor y, Tensor dy, Tensor(a!) rowdots, Tensor expert_rows, int EL) -> ()", &pfb::ep_row_dots);
  m.def("ep_pull_scalars(Tensor(a!) dots, Tensor idx, Tensor pair_slot, Tensor w, Tensor peer_rowdots_ptrs, int EL, int ep, "
        "int capacity_rows) -> ()", &pfb::ep_pull_scalars);
  m.def("ep_exchange(Tensor peer_tab_ptrs, Tensor my_counts, Tensor(a!) block_expert, Tensor(b!) expert_rows, Tensor(c!) total_rows, "
        "int rank, int ep, int EL, Tensor epoch, Tensor(d!)? expert_tot) -> ()", &pfb::ep_exchange);
  m.def("ep_zero_padding(Tensor(a!) buf, Tensor expert_rows, Tensor expert_tot, int EL) -> ()", &pfb::ep_zero_padding);
  m.def("ep_push_rows(Tensor x, Tensor idx, Tensor rank_in_expert, Tensor? scale, Tensor peer_tab_ptrs, Tensor(a!) pair_slot, "
        "Tensor peer_buf_ptrs, int k, int EL, int ep, int capacity_rows, int rank, int flag_slot, Tensor epoch, Tensor(b!) done_counter, "
        "bool slots_from_table) -> ()",
        &pfb::ep_push_rows);
  m.def("ep_wait_flag(Tensor peer_tab_ptrs, int rank, int ep, int EL, int flag_slot, Tensor epoch) -> ()", &pfb::ep_wait_flag);
  m.def("ep_signal_flag(Tensor peer_tab_ptrs, int rank, int ep, int EL, int flag_slot, Tensor epoch) -> ()", &pfb::ep_signal_flag);
  m.def("ep_pull_rows(Tensor(a!)? out, Tensor idx, Tensor pair_slot, Tensor? w, Tensor? g, Tensor(b!)? dots, Tensor peer_buf_ptrs, "
        "Tensor peer_tab_ptrs, int T, int k, int H, int EL, int ep, int capacity_rows) -> ()", &pfb::ep_pull_rows);
}
