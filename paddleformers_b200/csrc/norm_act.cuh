// Memory-bound fused kernels: RMSNorm (+residual add) fwd/bwd, SwiGLU fwd/bwd, RoPE (+per-head QK RMSNorm).
// All of them move 16 bytes per thread per access and keep every reduction in fp32.
//
// Counterparts in the reference: fused_rms_norm_ext (paddleformers/nn/norm.py:54-83), swiglu
// (paddleformers/nn/mlp.py:17-24), rotary embedding math (paddleformers/transformers/llama/modeling.py:40-67),
// partial rotary (paddleformers/transformers/glm4_moe/modeling.py:135-153).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pfb {

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ float warp_sum(float v) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is a shared array of >= 32 floats. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = l < nw ? red[l] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = l < nw ? red[l] : -INFINITY;
  return warp_max(r);
}

// y = rmsnorm(x (+ residual)) * w. If `residual` != nullptr the sum is also written to `sum_out`
// (pre-norm residual stream). One block per row; H % 8 == 0.
__global__ void rms_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                    __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd_out, int H,
                                    long long x_stride, long long y_stride, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * x_stride);
  const bf16x8* rr = residual ? reinterpret_cast<const bf16x8*>(residual + row * static_cast<long long>(H)) : nullptr;
  bf16x8* sr = sum_out ? reinterpret_cast<bf16x8*>(sum_out + row * static_cast<long long>(H)) : nullptr;
  const int nv = H >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    bf16x8 a = xr[i];
    if (rr) {
      bf16x8 b = rr[i];
      #pragma unroll
      for (int j = 0; j < 4; ++j) a.v[j] = __float22bfloat162_rn(make_float2(
          __low2float(a.v[j]) + __low2float(b.v[j]), __high2float(a.v[j]) + __high2float(b.v[j])));
      sr[i] = a;
    }
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a.v[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const bf16x8* src = rr ? reinterpret_cast<const bf16x8*>(sr) : xr;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * y_stride);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    bf16x8 a = src[i], ww = wr[i], o;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a.v[j]), g = __bfloat1622float2(ww.v[j]);
      o.v[j] = __float22bfloat162_rn(make_float2(f.x * rstd * g.x, f.y * rstd * g.y));
    }
    yr[i] = o;
  }
}

// dx = rstd * (dy*w) - x * rstd^3 * mean(dy*w*x)  (+ dres if given: gradient flowing through the residual stream)
// dw partials: each block owns rows blockIdx.x, +gridDim.x, ... and writes its partial sum to
// dw_partial[blockIdx.x, H] (fp32 scratch); rms_norm_dw_reduce_kernel folds the partials.
// blockDim.x * 8 * PER_THREAD >= H is required (PER_THREAD chunks of 8 columns per thread).
template <int PER_THREAD>
__global__ void __launch_bounds__(256, PER_THREAD <= 2 ? 4 : 1) rms_norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                    const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                                    const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                    float* __restrict__ dw_partial, int T, int H, long long dy_stride) {
  __shared__ float red[32];
  const int nv = H >> 3;
  float dwacc[PER_THREAD][8];
  #pragma unroll
  for (int c = 0; c < PER_THREAD; ++c)
    #pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[c][j] = 0.f;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + row * dy_stride);
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * static_cast<long long>(H));
    const float rstd = rstd_in[row];
    float dot = 0.f;
    float g[PER_THREAD][8], xv[PER_THREAD][8];
    #pragma unroll
    for (int c = 0; c < PER_THREAD; ++c) {
      const int i = threadIdx.x + c * blockDim.x;
      if (i < nv) {
        bf16x8 a = dyr[i], b = xr[i], ww = wr[i];
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 fa = __bfloat1622float2(a.v[j]), fb = __bfloat1622float2(b.v[j]), fw = __bfloat1622float2(ww.v[j]);
          g[c][2 * j] = fa.x * fw.x; g[c][2 * j + 1] = fa.y * fw.y;
          xv[c][2 * j] = fb.x; xv[c][2 * j + 1] = fb.y;
          dot += g[c][2 * j] * fb.x + g[c][2 * j + 1] * fb.y;
          dwacc[c][2 * j] += fa.x * fb.x * rstd; dwacc[c][2 * j + 1] += fa.y * fb.y * rstd;
        }
      }
    }
    dot = block_sum(dot, red);
    const float coef = dot * rstd * rstd * rstd / H;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * static_cast<long long>(H));
    const bf16x8* drr = dres ? reinterpret_cast<const bf16x8*>(dres + row * static_cast<long long>(H)) : nullptr;
    #pragma unroll
    for (int c = 0; c < PER_THREAD; ++c) {
      const int i = threadIdx.x + c * blockDim.x;
      if (i < nv) {
        bf16x8 o, r;
        if (drr) r = drr[i];
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a0 = rstd * g[c][2 * j] - coef * xv[c][2 * j];
          float a1 = rstd * g[c][2 * j + 1] - coef * xv[c][2 * j + 1];
          if (drr) { float2 fr = __bfloat1622float2(r.v[j]); a0 += fr.x; a1 += fr.y; }
          o.v[j] = __float22bfloat162_rn(make_float2(a0, a1));
        }
        dxr[i] = o;
      }
    }
  }
  #pragma unroll
  for (int c = 0; c < PER_THREAD; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nv) {
      float4* dst = reinterpret_cast<float4*>(dw_partial + static_cast<long long>(blockIdx.x) * H + i * 8);
      dst[0] = make_float4(dwacc[c][0], dwacc[c][1], dwacc[c][2], dwacc[c][3]);
      dst[1] = make_float4(dwacc[c][4], dwacc[c][5], dwacc[c][6], dwacc[c][7]);
    }
  }
}

// dw[h] (+)= sum_p partial[p, h]; accumulate != 0 adds to the existing fp32 value (main_grad semantics).
// One block of 256 threads per 32 columns: 8 row groups read 128-byte lines, each with 4 independent partial sums; the
// groups are combined through shared memory in a fixed order.
__global__ void rms_norm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int P, int H,
                                          int accumulate) {
  __shared__ float red[8][33];
  const int col = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int h = blockIdx.x * 32 + col;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (h < H) {
    int p = grp;
    for (; p + 24 < P; p += 32) {
      s0 += partial[static_cast<long long>(p) * H + h];
      s1 += partial[static_cast<long long>(p + 8) * H + h];
      s2 += partial[static_cast<long long>(p + 16) * H + h];
      s3 += partial[static_cast<long long>(p + 24) * H + h];
    }
    for (; p < P; p += 8) s0 += partial[static_cast<long long>(p) * H + h];
  }
  red[grp][col] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (grp == 0 && h < H) {
    float s = 0.f;
    #pragma unroll
    for (int g = 0; g < 8; ++g) s += red[g][col];
    dw[h] = accumulate ? dw[h] + s : s;
  }
}

// act[t, i] = silu(gu[t, i]) * gu[t, I + i]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, long long T,
                                  int I, long long gu_stride) {
  const int nv = I >> 3;
  const long long total = T * nv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / nv;
    const int i = static_cast<int>(idx - t * nv);
    const bf16x8 g = reinterpret_cast<const bf16x8*>(gu + t * gu_stride)[i];
    const bf16x8 u = reinterpret_cast<const bf16x8*>(gu + t * gu_stride + I)[i];
    bf16x8 o;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fg = __bfloat1622float2(g.v[j]), fu = __bfloat1622float2(u.v[j]);
      o.v[j] = __float22bfloat162_rn(make_float2(fg.x / (1.f + __expf(-fg.x)) * fu.x, fg.y / (1.f + __expf(-fg.y)) * fu.y));
    }
    reinterpret_cast<bf16x8*>(act + t * static_cast<long long>(I))[i] = o;
  }
}

// dgu = [dact * u * silu'(g), dact * silu(g)]; optionally recomputes act (for the down-proj wgrad) and applies a
// per-row probability `prob` (MoE weighted SwiGLU: act = prob * silu(g) * u, returns dprob by atomics-free row sums
// when dprob != nullptr; in that mode one warp handles one row).
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dact, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, __nv_bfloat16* __restrict__ act_out, long long T,
                                  int I, long long gu_stride) {
  const int nv = I >> 3;
  const long long total = T * nv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / nv;
    const int i = static_cast<int>(idx - t * nv);
    const bf16x8 g = reinterpret_cast<const bf16x8*>(gu + t * gu_stride)[i];
    const bf16x8 u = reinterpret_cast<const bf16x8*>(gu + t * gu_stride + I)[i];
    const bf16x8 d = reinterpret_cast<const bf16x8*>(dact + t * static_cast<long long>(I))[i];
    bf16x8 og, ou, oa;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fg = __bfloat1622float2(g.v[j]), fu = __bfloat1622float2(u.v[j]), fd = __bfloat1622float2(d.v[j]);
      float s0 = 1.f / (1.f + __expf(-fg.x)), s1 = 1.f / (1.f + __expf(-fg.y));
      float si0 = fg.x * s0, si1 = fg.y * s1;
      og.v[j] = __float22bfloat162_rn(make_float2(fd.x * fu.x * (s0 + si0 * (1.f - s0)), fd.y * fu.y * (s1 + si1 * (1.f - s1))));
      ou.v[j] = __float22bfloat162_rn(make_float2(fd.x * si0, fd.y * si1));
      oa.v[j] = __float22bfloat162_rn(make_float2(si0 * fu.x, si1 * fu.y));
    }
    reinterpret_cast<bf16x8*>(dgu + t * 2LL * I)[i] = og;
    reinterpret_cast<bf16x8*>(dgu + t * 2LL * I + I)[i] = ou;
    if (act_out) reinterpret_cast<bf16x8*>(act_out + t * static_cast<long long>(I))[i] = oa;
  }
}

// In-place rotary embedding on a [T, n_heads, D] strided view (row stride `row_stride`, head stride D):
//   out[:rot/2] = x1*cos - x2*sin ; out[rot/2:rot] = x2*cos + x1*sin, with x1 = x[:rot/2], x2 = x[rot/2:rot].
// `sign` = -1 gives the backward (conjugate) rotation. cos/sin are fp32 [n_pos, rot/2], indexed by pos[t].
// Optional per-head RMSNorm over D (weight `nw`) applied before the rotation (QK-norm); in that mode
// `rstd_out[t, head]` is saved for the backward pass and the input is read from `x` and written to `out`.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ cs,
                            const float* __restrict__ sn, int T, int n_heads, int D, int rot, long long row_stride,
                            float sign) {
  const int half = rot >> 1;
  const int pairs_per_row = n_heads * half;
  const long long total = static_cast<long long>(T) * pairs_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / pairs_per_row);
    const int r = static_cast<int>(idx - static_cast<long long>(t) * pairs_per_row);
    const int h = r / half, i = r - h * half;
    const int p = pos ? pos[t] : t;
    const float c = cs[static_cast<long long>(p) * half + i], s = sign * sn[static_cast<long long>(p) * half + i];
    __nv_bfloat16* base = x + t * row_stride + static_cast<long long>(h) * D;
    const float x1 = __bfloat162float(base[i]), x2 = __bfloat162float(base[i + half]);
    base[i] = __float2bfloat16(x1 * c - x2 * s);
    base[i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
}

// The same rotation with 16-byte accesses: one thread rotates 8 adjacent pairs (x1[i..i+8), x2[i..i+8)). Needs
// rot % 16 == 0, D % 8 == 0, row_stride % 8 == 0 and a 16-byte aligned base.
__global__ void rope_vec8_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ cs,
                                 const float* __restrict__ sn, int T, int n_heads, int D, int rot, long long row_stride,
                                 float sign) {
  const int half = rot >> 1, hv = half >> 3;
  const int per_row = n_heads * hv;
  const long long total = static_cast<long long>(T) * per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(idx / per_row);
    const int r = static_cast<int>(idx - static_cast<long long>(t) * per_row);
    const int h = r / hv, i = (r - h * hv) * 8;
    const int p = pos ? pos[t] : t;
    const float4* c4 = reinterpret_cast<const float4*>(cs + static_cast<long long>(p) * half + i);
    const float4* s4 = reinterpret_cast<const float4*>(sn + static_cast<long long>(p) * half + i);
    const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    const float c[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    const float sv[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    __nv_bfloat16* base = x + t * row_stride + static_cast<long long>(h) * D + i;
    const bf16x8 a = *reinterpret_cast<const bf16x8*>(base), b = *reinterpret_cast<const bf16x8*>(base + half);
    bf16x8 oa, ob;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f1 = __bfloat1622float2(a.v[j]), f2 = __bfloat1622float2(b.v[j]);
      const float s0 = sign * sv[2 * j], s1 = sign * sv[2 * j + 1];
      oa.v[j] = __float22bfloat162_rn(make_float2(f1.x * c[2 * j] - f2.x * s0, f1.y * c[2 * j + 1] - f2.y * s1));
      ob.v[j] = __float22bfloat162_rn(make_float2(f2.x * c[2 * j] + f1.x * s0, f2.y * c[2 * j + 1] + f1.y * s1));
    }
    *reinterpret_cast<bf16x8*>(base) = oa;
    *reinterpret_cast<bf16x8*>(base + half) = ob;
  }
}

// One warp per (token, head): y = rmsnorm_D(x) * nw, then rotary on the first `rot` dims. D <= 256, D % 64 == 0 not
// required (D % 2 == 0). Out-of-place so that the backward can re-read x.
__global__ void qk_norm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                        const __nv_bfloat16* __restrict__ nw, float* __restrict__ rstd_out,
                                        const int* __restrict__ pos, const float* __restrict__ cs,
                                        const float* __restrict__ sn, int T, int n_heads, int D, int rot,
                                        long long x_row_stride, long long out_row_stride, float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T * n_heads) return;
  const int t = warp / n_heads, h = warp - t * n_heads;
  const __nv_bfloat16* xin = x + t * x_row_stride + static_cast<long long>(h) * D;
  __nv_bfloat16* o = out + t * out_row_stride + static_cast<long long>(h) * D;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) { float v = __bfloat162float(xin[i]); ss += v * v; }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / D + eps);
  if (lane == 0 && rstd_out) rstd_out[warp] = rstd;
  const int half = rot >> 1;
  const int p = pos ? pos[t] : t;
  for (int i = lane; i < half; i += 32) {
    const float c = cs[static_cast<long long>(p) * half + i], s = sn[static_cast<long long>(p) * half + i];
    const float x1 = __bfloat162float(xin[i]) * rstd * __bfloat162float(nw[i]);
    const float x2 = __bfloat162float(xin[i + half]) * rstd * __bfloat162float(nw[i + half]);
    o[i] = __float2bfloat16(x1 * c - x2 * s);
    o[i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
  for (int i = rot + lane; i < D; i += 32)
    o[i] = __float2bfloat16(__bfloat162float(xin[i]) * rstd * __bfloat162float(nw[i]));
}

// Backward of qk_norm_rope: un-rotate dout, then RMSNorm backward over D. Warps stride over (token, head) pairs
// and keep their dnw contribution in registers; one shared-memory reduction and D global atomics per block.
__global__ void qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ x,
                                        const __nv_bfloat16* __restrict__ nw, const float* __restrict__ rstd_in,
                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dnw,
                                        const int* __restrict__ pos, const float* __restrict__ cs,
                                        const float* __restrict__ sn, int T, int n_heads, int D, int rot,
                                        long long dout_row_stride, long long x_row_stride, long long dx_row_stride) {
  __shared__ float sdnw[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) sdnw[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_total = (gridDim.x * blockDim.x) >> 5;
  const int half = rot >> 1;
  float dnw_acc[8];
  #pragma unroll
  for (int k = 0; k < 8; ++k) dnw_acc[k] = 0.f;
  for (int wi = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; wi < T * n_heads; wi += warps_total) {
    const int t = wi / n_heads, h = wi - t * n_heads;
    const __nv_bfloat16* dor = dout + t * dout_row_stride + static_cast<long long>(h) * D;
    const __nv_bfloat16* xin = x + t * x_row_stride + static_cast<long long>(h) * D;
    __nv_bfloat16* dxo = dx + t * dx_row_stride + static_cast<long long>(h) * D;
    const float rstd = rstd_in[wi];
    const int p = pos ? pos[t] : t;
    float dyv[8], xv[8];
    float dot = 0.f;
    #pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = lane + 32 * k;
      dyv[k] = 0.f; xv[k] = 0.f;
      if (i < D) {
        float d;
        if (i < rot) {
          const int ii = i < half ? i : i - half;
          const float c = cs[static_cast<long long>(p) * half + ii], s = sn[static_cast<long long>(p) * half + ii];
          const float d1 = __bfloat162float(dor[ii]), d2 = __bfloat162float(dor[ii + half]);
          d = i < half ? (d1 * c + d2 * s) : (d2 * c - d1 * s);
        } else {
          d = __bfloat162float(dor[i]);
        }
        xv[k] = __bfloat162float(xin[i]);
        dnw_acc[k] += d * xv[k] * rstd;
        dyv[k] = d * __bfloat162float(nw[i]);
        dot += dyv[k] * xv[k];
      }
    }
    dot = warp_sum(dot);
    const float coef = dot * rstd * rstd * rstd / D;
    #pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = lane + 32 * k;
      if (i < D) dxo[i] = __float2bfloat16(rstd * dyv[k] - coef * xv[k]);
    }
  }
  #pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = lane + 32 * k;
    if (i < D) atomicAdd(&sdnw[i], dnw_acc[k]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dnw[i], sdnw[i]);
}

// ---- 128-wide heads with full rotary (D == rot == 128): 8-byte accesses -------------------------------------------
// Lane l holds elements 4l .. 4l+3 of the head; the rotation partner of element i (i + 64 or i - 64) lives in lane l ^ 16.
__device__ __forceinline__ void ld_bf16x4(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void st_bf16x4(__nv_bfloat16* p, const float (&f)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

__global__ void qk_norm_rope_fwd128_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                           const __nv_bfloat16* __restrict__ nw, float* __restrict__ rstd_out,
                                           const int* __restrict__ pos, const float* __restrict__ cs, const float* __restrict__ sn,
                                           int T, int n_heads, long long x_row_stride, long long out_row_stride, float eps) {
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(T) * n_heads;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  float w[4];
  ld_bf16x4(nw + lane * 4, w);
  const bool first = lane < 16;
  for (long long wi = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; wi < total; wi += warps_total) {
    const int t = static_cast<int>(wi / n_heads), h = static_cast<int>(wi - static_cast<long long>(t) * n_heads);
    float v[4];
    ld_bf16x4(x + t * x_row_stride + static_cast<long long>(h) * 128 + lane * 4, v);
    float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss * (1.f / 128.f) + eps);
    if (lane == 0 && rstd_out) rstd_out[wi] = rstd;
    const int p = pos ? pos[t] : t;
    const float4 c4 = *reinterpret_cast<const float4*>(cs + static_cast<long long>(p) * 64 + (lane & 15) * 4);
    const float4 s4 = *reinterpret_cast<const float4*>(sn + static_cast<long long>(p) * 64 + (lane & 15) * 4);
    const float c[4] = {c4.x, c4.y, c4.z, c4.w}, s[4] = {s4.x, s4.y, s4.z, s4.w};
    float o[4];
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float y = v[j] * rstd * w[j];
      const float other = __shfl_xor_sync(0xffffffffu, y, 16);
      o[j] = first ? y * c[j] - other * s[j] : y * c[j] + other * s[j];
    }
    st_bf16x4(out + t * out_row_stride + static_cast<long long>(h) * 128 + lane * 4, o);
  }
}

__global__ void qk_norm_rope_bwd128_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ x,
                                           const __nv_bfloat16* __restrict__ nw, const float* __restrict__ rstd_in,
                                           __nv_bfloat16* __restrict__ dx, float* __restrict__ dnw, const int* __restrict__ pos,
                                           const float* __restrict__ cs, const float* __restrict__ sn, int T, int n_heads,
                                           long long dout_row_stride, long long x_row_stride, long long dx_row_stride) {
  __shared__ float sdnw[128];
  for (int i = threadIdx.x; i < 128; i += blockDim.x) sdnw[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(T) * n_heads;
  const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  float w[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
  ld_bf16x4(nw + lane * 4, w);
  const bool first = lane < 16;
  for (long long wi = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; wi < total; wi += warps_total) {
    const int t = static_cast<int>(wi / n_heads), h = static_cast<int>(wi - static_cast<long long>(t) * n_heads);
    float d[4], xv[4];
    ld_bf16x4(dout + t * dout_row_stride + static_cast<long long>(h) * 128 + lane * 4, d);
    ld_bf16x4(x + t * x_row_stride + static_cast<long long>(h) * 128 + lane * 4, xv);
    const float rstd = rstd_in[wi];
    const int p = pos ? pos[t] : t;
    const float4 c4 = *reinterpret_cast<const float4*>(cs + static_cast<long long>(p) * 64 + (lane & 15) * 4);
    const float4 s4 = *reinterpret_cast<const float4*>(sn + static_cast<long long>(p) * 64 + (lane & 15) * 4);
    const float c[4] = {c4.x, c4.y, c4.z, c4.w}, s[4] = {s4.x, s4.y, s4.z, s4.w};
    float dy[4], dot = 0.f;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, d[j], 16);
      const float g = first ? d[j] * c[j] + other * s[j] : d[j] * c[j] - other * s[j];   // gradient of the normed, weighted value
      acc[j] += g * xv[j] * rstd;
      dy[j] = g * w[j];
      dot += dy[j] * xv[j];
    }
    dot = warp_sum(dot);
    const float coef = dot * rstd * rstd * rstd * (1.f / 128.f);
    float o[4];
    #pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = rstd * dy[j] - coef * xv[j];
    st_bf16x4(dx + t * dx_row_stride + static_cast<long long>(h) * 128 + lane * 4, o);
  }
  #pragma unroll
  for (int j = 0; j < 4; ++j) atomicAdd(&sdnw[lane * 4 + j], acc[j]);
  __syncthreads();
  for (int i = threadIdx.x; i < 128; i += blockDim.x) atomicAdd(&dnw[i], sdnw[i]);
}

}  // namespace pfb
