// Cross-entropy over a chunk of bf16 logits (loss + in-place gradient), embedding gather / scatter-add,
// fused AdamW on flat fp32 master buffers, squared-norm reduction, cast/scale helpers.
//
// Counterparts in the reference: the chunked fused head + cross entropy
// (paddleformers/transformers/tensor_parallel_utils.py:133-569), AdamW math
// (paddleformers/utils/optimizer.py:573-600, paddleformers/utils/adamw_triton.py:39-138), global-norm clipping
// (paddleformers/utils/moe_hybrid_parallel_optimizer.py:162-389), embedding grad add
// (paddleformers/cli/train/deepseek_v3_pretrain/modeling_pp.py:1447-1456).
#pragma once
#include "norm_act.cuh"

namespace pfb {

// One block per row of logits [rows, V] (bf16, row stride ld). Computes
//   loss[row] = logsumexp(logits) - logits[label]            (0 when label == ignore_index)
// and overwrites the row with grad_scale[0] * (softmax - onehot) (0 rows for ignored labels), in bf16.
// `vocab_start` / `V` describe the vocabulary shard this tensor holds; with a shard (tensor parallel) the caller
// passes the already all-reduced row max and sum in `g_max`, `g_sum` and this kernel only writes gradients
// (mode 2). Mode 0: single-shard fused loss+grad. Mode 1: write local (max, sumexp(max), label logit) partials.
__global__ void cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                                     float* __restrict__ loss, float* __restrict__ stat_max,
                                     float* __restrict__ stat_sum, float* __restrict__ stat_label,
                                     const float* __restrict__ grad_scale, int V, long long ld, int vocab_start,
                                     long long ignore_index, int mode, int write_grad) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = label == ignore_index;
  const int nv = V >> 3;  // V % 8 == 0
  const long long local = label - vocab_start;
  float mx, sum;
  if (mode != 2) {
    mx = -INFINITY;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      bf16x8 a = reinterpret_cast<const bf16x8*>(lr)[i];
      #pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(a.v[j]); mx = fmaxf(mx, fmaxf(f.x, f.y)); }
    }
    mx = block_max(mx, red);
    sum = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      bf16x8 a = reinterpret_cast<const bf16x8*>(lr)[i];
      #pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(a.v[j]); sum += __expf(f.x - mx) + __expf(f.y - mx); }
    }
    sum = block_sum(sum, red);
    const float lab = (!ignored && local >= 0 && local < V) ? __bfloat162float(lr[local]) : 0.f;
    if (mode == 1) {
      if (threadIdx.x == 0) { stat_max[row] = mx; stat_sum[row] = sum; stat_label[row] = lab; }
      return;
    }
    if (threadIdx.x == 0) loss[row] = ignored ? 0.f : (logf(sum) + mx - lab);
  } else {
    mx = stat_max[row];
    sum = stat_sum[row];
  }
  if (!write_grad) return;
  const float scale = ignored ? 0.f : grad_scale[0];
  const float inv = 1.f / sum;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    bf16x8 a = reinterpret_cast<const bf16x8*>(lr)[i], o;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a.v[j]);
      float p0 = __expf(f.x - mx) * inv, p1 = __expf(f.y - mx) * inv;
      const int c = i * 8 + 2 * j;
      if (c == local) p0 -= 1.f;
      if (c + 1 == local) p1 -= 1.f;
      o.v[j] = __float22bfloat162_rn(make_float2(p0 * scale, p1 * scale));
    }
    reinterpret_cast<bf16x8*>(lr)[i] = o;
  }
}

// out[t, :] = W[ids[t] - vocab_start, :] (zeros when the id falls outside this vocabulary shard)
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ W,
                                     __nv_bfloat16* __restrict__ out, int T, int H, int vocab_start, int vocab_rows) {
  const int nv = H >> 3;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < static_cast<long long>(T) * nv;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / nv), i = static_cast<int>(idx - static_cast<long long>(t) * nv);
    const long long id = ids[t] - vocab_start;
    bf16x8 v;
    if (id >= 0 && id < vocab_rows) v = reinterpret_cast<const bf16x8*>(W + id * H)[i];
    else {
      #pragma unroll
      for (int j = 0; j < 4; ++j) v.v[j] = __float2bfloat162_rn(0.f);
    }
    reinterpret_cast<bf16x8*>(out + static_cast<long long>(t) * H)[i] = v;
  }
}

// main_grad[ids[t] - vocab_start, :] += dout[t, :]   (fp32 atomics; rows hit by several tokens add up)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ grad, int T, int H, int vocab_start, int vocab_rows) {
  const int nv = H >> 1;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < static_cast<long long>(T) * nv;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / nv), i = static_cast<int>(idx - static_cast<long long>(t) * nv);
    const long long id = ids[t] - vocab_start;
    if (id < 0 || id >= vocab_rows) continue;
    const float2 f = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(dout + static_cast<long long>(t) * H)[i]);
    float* g = grad + id * H + 2 * i;
    atomicAdd(g, f.x);
    atomicAdd(g + 1, f.y);
  }
}

// Decoupled AdamW on a flat shard: fp32 master p, moments m, v, fp32 gradient g; writes the bf16 working copy.
// `scalars` (device, fp32): [0] = lr, [1] = gradient multiplier (clip coefficient * 1/loss-scale),
// [2] = 1 - beta1^t, [3] = 1 - beta2^t, [4] = skip flag (non-zero: leave everything untouched, e.g. inf/nan step).
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ g, __nv_bfloat16* __restrict__ p16, long long n,
                             const float* __restrict__ scalars, float beta1, float beta2, float eps, float wd) {
  if (scalars[4] != 0.f) return;
  const float lr = scalars[0], gmul = scalars[1], bc1 = scalars[2], bc2 = scalars[3];
  const long long nv = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i], mm = reinterpret_cast<float4*>(m)[i],
           vv = reinterpret_cast<float4*>(v)[i], gg = reinterpret_cast<const float4*>(g)[i];
    float* P = reinterpret_cast<float*>(&pp); float* Mm = reinterpret_cast<float*>(&mm);
    float* Vv = reinterpret_cast<float*>(&vv); float* G = reinterpret_cast<float*>(&gg);
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = G[j] * gmul;
      Mm[j] = beta1 * Mm[j] + (1.f - beta1) * gr;
      Vv[j] = beta2 * Vv[j] + (1.f - beta2) * gr * gr;
      const float mhat = Mm[j] / bc1, vhat = Vv[j] / bc2;
      P[j] = P[j] * (1.f - lr * wd) - lr * mhat / (sqrtf(vhat) + eps);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p16) {
      uint2 o;
      __nv_bfloat162 a = __float22bfloat162_rn(make_float2(P[0], P[1])), b = __float22bfloat162_rn(make_float2(P[2], P[3]));
      o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
      reinterpret_cast<uint2*>(p16)[i] = o;
    }
  }
  // tail (n % 4)
  const long long tail0 = nv << 2;
  for (long long i = tail0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gr = g[i] * gmul;
    m[i] = beta1 * m[i] + (1.f - beta1) * gr;
    v[i] = beta2 * v[i] + (1.f - beta2) * gr * gr;
    p[i] = p[i] * (1.f - lr * wd) - lr * (m[i] / bc1) / (sqrtf(v[i] / bc2) + eps);
    if (p16) p16[i] = __float2bfloat16(p[i]);
  }
}

// partial[blockIdx.x] = sum of squares of this block's grid-stride slice; sq_norm_finish adds the partials into
// out[0] (out must be zeroed by the caller when starting a new norm; several buffers may add into one scalar).
__global__ void sq_norm_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const long long nv = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 a = reinterpret_cast<const float4*>(x)[i];
    s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  for (long long i = (nv << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) s += x[i] * x[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void sq_norm_finish_kernel(const float* __restrict__ partial, int P, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] += s;
}

// dst(bf16) = src(fp32) * scale  /  dst(fp32) (+)= src(bf16) * scale
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                                        float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) dst[i] = __float2bfloat16(src[i] * scale);
}
__global__ void accum_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n,
                                         float scale, int accumulate) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = __bfloat162float(src[i]) * scale;
    dst[i] = accumulate ? dst[i] + v : v;
  }
}

}  // namespace pfb
