// Fused MoE routing for sm_100a: scores -> (group-limited, bias-corrected) top-k -> combine weights -> per-expert
// histogram -> stable rank of every (token, slot) pair inside its expert -> balance-loss statistics, in two launches
// instead of the few dozen tensor operations the same steps take when written with sort / cumsum / scatter.
//
//   moe_route_fwd   one warp per token (E <= 256 experts, lane L holds experts L, L + 32, ...): softmax or sigmoid
//                   scores, optional selection bias (aux-loss-free balancing), optional group limiting (groups of 32*m
//                   experts scored by their maximum or by the sum of their two best), k rounds of warp arg-max, combine
//                   weights (optionally normalised over the k, times a scale). Every CTA owns a contiguous run of
//                   tokens and records its own per-expert pair counts (for the rank pass) and the per-expert sums of
//                   the routing probabilities (for the balance loss).
//   moe_route_rank  the pairs of a CTA's token run are ranked in order (a warp walks them 32 at a time and uses
//                   match.any to rank equal experts inside a chunk), on top of the counts of all earlier runs: the
//                   result equals a stable sort by expert, without sorting. CTA 0 also adds up the total counts.
//   moe_route_bwd   d(logits) from d(combine weights) and from the balance loss (whose gradient per probability is a
//                   per-expert constant), recomputing the scores from the logits.
//
// Semantics follow the reference's gate: paddleformers/nn/moe_deepep/moe_gate.py:275-362 (top-k, group limits, bias),
// :126-158 and :464-499 (balance statistics), and the permutation bookkeeping of
// paddleformers/transformers/token_dispatcher.py:70-196.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "status.h"

namespace pfb {

constexpr int RT_MAX_PER_LANE = 8;     // E <= 256
constexpr int RT_WARPS = 8;            // warps per CTA
constexpr int RT_TOKENS_PER_CTA = 64;  // contiguous token run of one CTA (the unit of the rank pass)

struct RouteParams {
  const float* logits;   // [T, E]
  const float* sel_bias; // [E] or nullptr: added to the scores for SELECTION only
  long long* idx;        // [T, k]
  float* w;              // [T, k]
  int* block_counts;     // [n_ctas, E]
  float* prob_sums;      // [E] += sum over tokens of the routing probability (balance loss), or nullptr
  int T, E, k;
  int sigmoid;           // 0 softmax, 1 sigmoid
  int n_group, topk_group, group_top2;
  int norm_topk;
  float scale;
};

__device__ __forceinline__ float warp_max(float v) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// scores of one token in registers: s[j] belongs to expert lane + 32 j. Returns the normaliser of the probabilities
// used by the balance loss (1 for softmax, sum of the sigmoid scores otherwise).
__device__ __forceinline__ float token_scores(const float* __restrict__ row, int E, int lane, bool sigmoid, float (&s)[RT_MAX_PER_LANE]) {
  const int per = E >> 5;
  float mx = -INFINITY;
  #pragma unroll
  for (int j = 0; j < RT_MAX_PER_LANE; ++j) {
    s[j] = j < per ? row[lane + 32 * j] : -INFINITY;
    mx = fmaxf(mx, s[j]);
  }
  if (sigmoid) {
    float sum = 0.f;
    #pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j) {
      s[j] = j < per ? 1.f / (1.f + __expf(-s[j])) : 0.f;
      sum += s[j];
    }
    return warp_sum(sum);
  }
  mx = warp_max(mx);
  float sum = 0.f;
  #pragma unroll
  for (int j = 0; j < RT_MAX_PER_LANE; ++j) {
    s[j] = j < per ? __expf(s[j] - mx) : 0.f;
    sum += s[j];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  #pragma unroll
  for (int j = 0; j < RT_MAX_PER_LANE; ++j) s[j] *= inv;
  return 1.f;
}

__global__ void __launch_bounds__(RT_WARPS * 32) moe_route_fwd_kernel(const RouteParams p) {
  __shared__ int s_cnt[256];
  __shared__ float s_prob[256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 256; i += blockDim.x) { s_cnt[i] = 0; s_prob[i] = 0.f; }
  __syncthreads();
  const int per = p.E >> 5;
  const int t0 = blockIdx.x * RT_TOKENS_PER_CTA;
  float acc_prob[RT_MAX_PER_LANE];
  #pragma unroll
  for (int j = 0; j < RT_MAX_PER_LANE; ++j) acc_prob[j] = 0.f;
  for (int tt = warp; tt < RT_TOKENS_PER_CTA; tt += RT_WARPS) {
    const int t = t0 + tt;
    if (t >= p.T) break;
    float s[RT_MAX_PER_LANE], sel[RT_MAX_PER_LANE];
    const float norm = token_scores(p.logits + static_cast<long long>(t) * p.E, p.E, lane, p.sigmoid != 0, s);
    const float inv_norm = 1.f / (norm + (p.sigmoid ? 1e-20f : 0.f));
    #pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j) {
      acc_prob[j] += s[j] * inv_norm;
      sel[j] = j < per ? s[j] + (p.sel_bias ? p.sel_bias[lane + 32 * j] : 0.f) : -INFINITY;
    }
    if (p.n_group > 1) {
      // group g = experts [g * gs, (g + 1) * gs), gs a multiple of 32: the registers j in [g * m, (g + 1) * m) of all lanes
      const int m = per / p.n_group;
      float gscore[RT_MAX_PER_LANE];
      #pragma unroll
      for (int g = 0; g < RT_MAX_PER_LANE; ++g) {
        gscore[g] = -INFINITY;
        if (g < p.n_group) {
          float best = -INFINITY, second = -INFINITY;
          #pragma unroll
          for (int j = 0; j < RT_MAX_PER_LANE; ++j) {       // static indices keep sel[] in registers
            if (j < per && j / m == g) {
              const float v = sel[j];
              if (v > best) { second = best; best = v; } else if (v > second) second = v;
            }
          }
          // merge the per-lane (best, second) pairs across the warp
          #pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, second, o);
            const float nb = fmaxf(best, ob);
            const float ns = fmaxf(fminf(best, ob), fmaxf(second, os));
            best = nb; second = ns;
          }
          gscore[g] = p.group_top2 ? best + second : best;
        }
      }
      // keep the topk_group best groups (ties: lower group index first)
      unsigned keep = 0;
      for (int r = 0; r < p.topk_group; ++r) {
        int bg = -1; float bv = -INFINITY;
        #pragma unroll
        for (int g = 0; g < RT_MAX_PER_LANE; ++g)
          if (g < p.n_group && !((keep >> g) & 1u) && (bg < 0 || gscore[g] > bv)) { bg = g; bv = gscore[g]; }
        keep |= 1u << bg;
      }
      #pragma unroll
      for (int j = 0; j < RT_MAX_PER_LANE; ++j)
        if (j < per && !((keep >> (j / m)) & 1u)) sel[j] = -INFINITY;
    }
    // k rounds of warp arg-max (ties: lower expert index first)
    float wsel = 0.f, wsum = 0.f;
    int my_e = -1;
    for (int r = 0; r < p.k; ++r) {
      float bv = -INFINITY; int be = 0x7fffffff;
      #pragma unroll
      for (int j = 0; j < RT_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        if (j < per && (sel[j] > bv || (sel[j] == bv && e < be))) { bv = sel[j]; be = e; }
      }
      #pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
      // the owner lane removes the winner and hands out its score; lane r keeps the round's result
      const int owner = be & 31, jj = be >> 5;
      float sc = 0.f;
      #pragma unroll
      for (int j = 0; j < RT_MAX_PER_LANE; ++j)
        if (lane == owner && j == jj) { sc = s[j]; sel[j] = -INFINITY; }
      sc = __shfl_sync(0xffffffffu, sc, owner);
      wsum += sc;
      if (lane == r) { my_e = be; wsel = sc; }
    }
    if (lane < p.k) {
      float wv = wsel;
      if (p.norm_topk && p.k > 1) wv = wv / (wsum + 1e-20f);
      wv *= p.scale;
      p.idx[static_cast<long long>(t) * p.k + lane] = my_e;
      p.w[static_cast<long long>(t) * p.k + lane] = wv;
      atomicAdd(&s_cnt[my_e], 1);
    }
  }
  // per-CTA statistics
  #pragma unroll
  for (int j = 0; j < RT_MAX_PER_LANE; ++j)
    if (j < per) atomicAdd(&s_prob[lane + 32 * j], acc_prob[j]);
  __syncthreads();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    p.block_counts[static_cast<long long>(blockIdx.x) * p.E + e] = s_cnt[e];
    if (p.prob_sums) atomicAdd(p.prob_sums + e, s_prob[e]);
  }
}

// rank_in_expert[pair] = number of earlier pairs (in pair order) routed to the same expert; counts[e] = total pairs.
__global__ void __launch_bounds__(256) moe_route_rank_kernel(const long long* __restrict__ idx, const int* __restrict__ block_counts,
                                                             int* __restrict__ rank_in_expert, int* __restrict__ counts,
                                                             long long* __restrict__ usage, int T, int E, int k, int n_ctas) {
  __shared__ int s_base[256];
  const int b = blockIdx.x;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int base = 0;
    for (int bb = 0; bb < b; ++bb) base += block_counts[static_cast<long long>(bb) * E + e];
    s_base[e] = base;
    if (b == n_ctas - 1) {
      const int total = base + block_counts[static_cast<long long>(b) * E + e];
      counts[e] = total;
      if (usage) usage[e] += total;
    }
  }
  __syncthreads();
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  const long long p0 = static_cast<long long>(b) * RT_TOKENS_PER_CTA * k;
  const long long p1 = min(static_cast<long long>(T) * k, p0 + static_cast<long long>(RT_TOKENS_PER_CTA) * k);
  for (long long q = p0; q < p1; q += 32) {
    const long long i = q + lane;
    const bool valid = i < p1;
    const int e = valid ? static_cast<int>(idx[i]) : -1 - lane;          // distinct keys for idle lanes
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int before = __popc(same & ((1u << lane) - 1u));
    int base = 0;
    if (valid) base = s_base[e];
    __syncwarp();
    if (valid) {
      rank_in_expert[i] = base + before;
      if (before == 0) s_base[e] = base + __popc(same);                 // the first lane of every group advances its expert
    }
    __syncwarp();
  }
}

struct RouteBwdParams {
  const float* logits; const float* sel_bias; const long long* idx; const float* dw; const float* aux_vec; float* dlogits;
  int T, E, k, sigmoid, norm_topk;
  float scale;
};

// d(logits)[t, :] from d(w)[t, :] and the balance term aux_vec[e] * prob[t, e] (aux_vec may be nullptr).
__global__ void __launch_bounds__(RT_WARPS * 32) moe_route_bwd_kernel(const RouteBwdParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = p.E >> 5;
  const long long t = static_cast<long long>(blockIdx.x) * RT_WARPS + warp;
  if (t >= p.T) return;
  float s[RT_MAX_PER_LANE], ds[RT_MAX_PER_LANE];
  const float norm = token_scores(p.logits + t * p.E, p.E, lane, p.sigmoid != 0, s);
  #pragma unroll
  for (int j = 0; j < RT_MAX_PER_LANE; ++j) ds[j] = 0.f;
  // combine weights: w_r = scale * s_r / (sum_sel s + eps) (or scale * s_r)
  float sum_sel = 0.f, dot = 0.f;
  int my_e = -1; float my_dw = 0.f, my_s = 0.f;
  if (lane < p.k) { my_e = static_cast<int>(p.idx[t * p.k + lane]); my_dw = p.dw[t * p.k + lane]; }
  #pragma unroll 1
  for (int r = 0; r < p.k; ++r) {
    const int e = __shfl_sync(0xffffffffu, my_e, r);
    float sc = 0.f;
    #pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j)
      if (lane == (e & 31) && j == (e >> 5)) sc = s[j];
    sc = __shfl_sync(0xffffffffu, sc, e & 31);
    if (lane == r) my_s = sc;
    sum_sel += sc;
    dot += __shfl_sync(0xffffffffu, my_dw, r) * sc;
  }
  if (lane < p.k) {
    float g;
    if (p.norm_topk && p.k > 1) {
      const float den = sum_sel + 1e-20f;
      g = p.scale * (my_dw / den - dot / (den * den));
    } else {
      g = p.scale * my_dw;
    }
    my_dw = g;   // d(score of the selected expert)
    (void)my_s;
  }
  #pragma unroll 1
  for (int r = 0; r < p.k; ++r) {
    const int e = __shfl_sync(0xffffffffu, my_e, r);
    const float g = __shfl_sync(0xffffffffu, my_dw, r);
    #pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j)
      if (lane == (e & 31) && j == (e >> 5)) ds[j] += g;
  }
  // balance loss: L = sum_e aux_vec[e] * prob[t, e], prob = s (softmax) or s / (sum s + eps) (sigmoid)
  if (p.aux_vec) {
    if (p.sigmoid) {
      const float den = norm + 1e-20f;
      float av = 0.f;
      #pragma unroll
      for (int j = 0; j < RT_MAX_PER_LANE; ++j) if (j < per) av += p.aux_vec[lane + 32 * j] * s[j];
      av = warp_sum(av);
      #pragma unroll
      for (int j = 0; j < RT_MAX_PER_LANE; ++j) if (j < per) ds[j] += p.aux_vec[lane + 32 * j] / den - av / (den * den);
    } else {
      #pragma unroll
      for (int j = 0; j < RT_MAX_PER_LANE; ++j) if (j < per) ds[j] += p.aux_vec[lane + 32 * j];
    }
  }
  // through the score function
  float* out = p.dlogits + t * p.E;
  if (p.sigmoid) {
    #pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j) if (j < per) out[lane + 32 * j] = ds[j] * s[j] * (1.f - s[j]);
  } else {
    float d = 0.f;
    #pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j) if (j < per) d += ds[j] * s[j];
    d = warp_sum(d);
    #pragma unroll
    for (int j = 0; j < RT_MAX_PER_LANE; ++j) if (j < per) out[lane + 32 * j] = s[j] * (ds[j] - d);
  }
}

// Returns (idx [T,k] int64, w [T,k] fp32, rank_in_expert [T*k] int32, counts [E] int32). prob_sums ([E] fp32, += ) and
// usage ([E] int64, += ) are optional accumulators.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> moe_route_fwd(
    const at::Tensor& logits, const c10::optional<at::Tensor>& sel_bias, int64_t k, bool sigmoid, int64_t n_group, int64_t topk_group,
    bool group_top2, bool norm_topk, double scale, c10::optional<at::Tensor> prob_sums, c10::optional<at::Tensor> usage) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == at::kFloat);
  const int T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(E % 32 == 0 && E <= 32 * RT_MAX_PER_LANE && k >= 1 && k <= 32 && k <= E, "moe_route: 32 | E <= 256, k <= 32");
  TORCH_CHECK(n_group >= 1 && (n_group == 1 || ((E / 32) % n_group == 0 && topk_group >= 1 && topk_group <= n_group)),
              "moe_route: expert groups must be multiples of 32 experts");
  const c10::cuda::CUDAGuard guard(logits.device());
  auto idx = at::empty({T, k}, logits.options().dtype(at::kLong));
  auto w = at::empty({T, k}, logits.options());
  auto rank = at::empty({T * k}, logits.options().dtype(at::kInt));
  auto counts = at::zeros({E}, logits.options().dtype(at::kInt));
  if (T == 0) return {idx, w, rank, counts};
  const int n_ctas = (T + RT_TOKENS_PER_CTA - 1) / RT_TOKENS_PER_CTA;
  auto block_counts = at::empty({n_ctas, E}, logits.options().dtype(at::kInt));
  RouteParams p;
  p.logits = logits.data_ptr<float>();
  p.sel_bias = nullptr;
  if (sel_bias.has_value()) {
    TORCH_CHECK(sel_bias->scalar_type() == at::kFloat && sel_bias->numel() == E && sel_bias->is_contiguous());
    p.sel_bias = sel_bias->data_ptr<float>();
  }
  p.idx = reinterpret_cast<long long*>(idx.data_ptr<int64_t>()); p.w = w.data_ptr<float>();
  p.block_counts = block_counts.data_ptr<int>();
  p.prob_sums = nullptr;
  if (prob_sums.has_value()) {
    TORCH_CHECK(prob_sums->scalar_type() == at::kFloat && prob_sums->numel() == E);
    p.prob_sums = prob_sums->data_ptr<float>();
  }
  p.T = T; p.E = E; p.k = k; p.sigmoid = sigmoid ? 1 : 0;
  p.n_group = n_group; p.topk_group = topk_group; p.group_top2 = group_top2 ? 1 : 0; p.norm_topk = norm_topk ? 1 : 0;
  p.scale = static_cast<float>(scale);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  moe_route_fwd_kernel<<<n_ctas, RT_WARPS * 32, 0, stream>>>(p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  long long* usage_ptr = nullptr;
  if (usage.has_value()) {
    TORCH_CHECK(usage->scalar_type() == at::kLong && usage->numel() == E);
    usage_ptr = reinterpret_cast<long long*>(usage->data_ptr<int64_t>());
  }
  moe_route_rank_kernel<<<n_ctas, 256, 0, stream>>>(p.idx, p.block_counts, rank.data_ptr<int>(), counts.data_ptr<int>(), usage_ptr, T, E,
                                                   static_cast<int>(k), n_ctas);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
  return {idx, w, rank, counts};
}

at::Tensor moe_route_bwd(const at::Tensor& logits, const c10::optional<at::Tensor>& sel_bias, const at::Tensor& idx, const at::Tensor& dw,
                         const c10::optional<at::Tensor>& aux_vec, bool sigmoid, bool norm_topk, double scale) {
  TORCH_CHECK(logits.is_cuda() && logits.is_contiguous() && logits.scalar_type() == at::kFloat && idx.scalar_type() == at::kLong);
  TORCH_CHECK(dw.scalar_type() == at::kFloat && dw.is_contiguous() && idx.is_contiguous() && dw.sizes() == idx.sizes());
  const int T = logits.size(0), E = logits.size(1), k = idx.size(1);
  const c10::cuda::CUDAGuard guard(logits.device());
  auto dlogits = at::empty_like(logits);
  if (T == 0) return dlogits;
  RouteBwdParams p;
  p.logits = logits.data_ptr<float>(); p.sel_bias = nullptr;
  p.idx = reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()); p.dw = dw.data_ptr<float>();
  p.aux_vec = nullptr;
  if (aux_vec.has_value()) {
    TORCH_CHECK(aux_vec->scalar_type() == at::kFloat && aux_vec->numel() == E && aux_vec->is_contiguous());
    p.aux_vec = aux_vec->data_ptr<float>();
  }
  p.dlogits = dlogits.data_ptr<float>();
  p.T = T; p.E = E; p.k = k; p.sigmoid = sigmoid ? 1 : 0; p.norm_topk = norm_topk ? 1 : 0; p.scale = static_cast<float>(scale);
  moe_route_bwd_kernel<<<(T + RT_WARPS - 1) / RT_WARPS, RT_WARPS * 32, 0, at::cuda::getCurrentCUDAStream()>>>(p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return dlogits;
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("moe_route_fwd(Tensor logits, Tensor? sel_bias, int k, bool sigmoid, int n_group, int topk_group, bool group_top2, "
        "bool norm_topk, float scale, Tensor(a!)? prob_sums, Tensor(b!)? usage) -> (Tensor, Tensor, Tensor, Tensor)", &pfb::moe_route_fwd);
  m.def("moe_route_bwd(Tensor logits, Tensor? sel_bias, Tensor idx, Tensor dw, Tensor? aux_vec, bool sigmoid, bool norm_topk, "
        "float scale) -> Tensor", &pfb::moe_route_bwd);
}
