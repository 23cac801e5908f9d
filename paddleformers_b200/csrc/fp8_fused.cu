// Fused producers of block-scaled fp8 operands:
//
//   swiglu_quant_fwd   act = prob * silu(gate) * up, quantised per 1x128 block in the same pass (no bf16 round trip)
//   swiglu_quant_bwd   d(gate, up) from d(act), in bf16 for the weight gradient and quantised per 1x128 block for the
//                      input-gradient GEMM, the recomputed activation and the per-row probability gradient
//   fp8_quant_transpose  x[T, K] -> x^T[K, T] e4m3 with one scale per 128 TOKENS: the operand layout of an fp8
//                      weight-gradient GEMM, whose contraction runs over tokens
//
// Counterparts in the reference: fused_weighted_swiglu_act_quant and fused_swiglu_probs_bwd
// (paddleformers/transformers/fp8_utils.py:984, 1050-1100), fused_transpose_split_quant / the wgrad operands of
// FP8GroupGemmMlpFunctionNode (fp8_utils.py:1011-1190).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <cuda_fp8.h>

#include "sm100_common.cuh"
#include "status.h"

namespace pfb {

__device__ __forceinline__ uint32_t quant4_e4m3(float a, float b, float c, float d, float inv) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a * inv, b * inv), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c * inv, d * inv), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}
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
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&f)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
}

// One warp per (row, 128-column block of the activation): q[R, I] e4m3, s_t[I/128, R]; act (bf16) optional.
__global__ void swiglu_quant_fwd_kernel(const __nv_bfloat16* __restrict__ gu, long long ld, const float* __restrict__ prob,
                                        uint8_t* __restrict__ q, float* __restrict__ s_t, __nv_bfloat16* __restrict__ act,
                                        long long R, int I, bool ue8m0) {
  const int lane = threadIdx.x & 31;
  const int nb = I / 128;
  const long long units = R * nb;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long u = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; u < units; u += warps) {
    const int kb = static_cast<int>(u % nb);
    const long long t = u / nb;
    float g[4], up[4], a[4];
    load4(gu + t * ld + kb * 128 + lane * 4, g);
    load4(gu + t * ld + I + kb * 128 + lane * 4, up);
    const float pr = prob ? prob[t] : 1.f;
    float amax = 0.f;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      a[j] = pr * g[j] / (1.f + __expf(-g[j])) * up[j];
      amax = fmaxf(amax, fabsf(a[j]));
    }
    const float scale = fp8_block_scale(warp_max(amax), ue8m0);
    *reinterpret_cast<uint32_t*>(q + t * I + kb * 128 + lane * 4) = quant4_e4m3(a[0], a[1], a[2], a[3], 1.f / scale);
    if (lane == 0) s_t[static_cast<long long>(kb) * R + t] = scale;
    if (act) store4(act + t * I + kb * 128 + lane * 4, a);
  }
}

// One warp per (row, 128-column block): with d = prob * dact,
//   dgate = d * up * silu'(gate), dup = d * silu(gate); dgu[R, 2I] bf16, gq[R, 2I] e4m3 + gs_t[2I/128, R];
//   act = prob * silu(gate) * up (optional, bf16); dprob_part[kb, row] = sum_i dact * silu(gate) * up (optional).
__global__ void swiglu_quant_bwd_kernel(const __nv_bfloat16* __restrict__ dact, const __nv_bfloat16* __restrict__ gu,
                                        long long ld, const float* __restrict__ prob, __nv_bfloat16* __restrict__ dgu,
                                        uint8_t* __restrict__ gq, float* __restrict__ gs_t, __nv_bfloat16* __restrict__ act,
                                        float* __restrict__ dprob_part, long long R, int I, bool ue8m0) {
  const int lane = threadIdx.x & 31;
  const int nb = I / 128;
  const long long units = R * nb;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long u = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; u < units; u += warps) {
    const int kb = static_cast<int>(u % nb);
    const long long t = u / nb;
    const int c = kb * 128 + lane * 4;
    float g[4], up[4], d[4], dg[4], du[4], a[4];
    load4(gu + t * ld + c, g);
    load4(gu + t * ld + I + c, up);
    load4(dact + t * I + c, d);
    const float pr = prob ? prob[t] : 1.f;
    float mg = 0.f, mu = 0.f, dot = 0.f;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j])), si = g[j] * s;
      dot += d[j] * si * up[j];
      const float dj = pr * d[j];
      dg[j] = dj * up[j] * (s + si * (1.f - s));
      du[j] = dj * si;
      a[j] = pr * si * up[j];
      mg = fmaxf(mg, fabsf(dg[j]));
      mu = fmaxf(mu, fabsf(du[j]));
    }
    const float sg = fp8_block_scale(warp_max(mg), ue8m0), su = fp8_block_scale(warp_max(mu), ue8m0);
    store4(dgu + t * 2LL * I + c, dg);
    store4(dgu + t * 2LL * I + I + c, du);
    *reinterpret_cast<uint32_t*>(gq + t * 2LL * I + c) = quant4_e4m3(dg[0], dg[1], dg[2], dg[3], 1.f / sg);
    *reinterpret_cast<uint32_t*>(gq + t * 2LL * I + I + c) = quant4_e4m3(du[0], du[1], du[2], du[3], 1.f / su);
    if (act) store4(act + t * I + c, a);
    if (dprob_part) dot = warp_sum(dot);
    if (lane == 0) {
      gs_t[static_cast<long long>(kb) * R + t] = sg;
      gs_t[static_cast<long long>(nb + kb) * R + t] = su;
      if (dprob_part) dprob_part[static_cast<long long>(kb) * R + t] = dot;
    }
  }
}

// Tile of 128 tokens x 64 channels per CTA of 256 threads. Thread (pair, part) holds 2 adjacent channels of 16 tokens;
// the channel maxima over the 128 tokens are combined through shared memory; the quantised bytes are staged in shared
// memory (16-byte chunks XOR-swizzled by channel pair) so that every channel row leaves as one 128-byte line.
// q_t[K, ldq] (ldq = tokens rounded up to 128, the tail zero-filled), s[T/128, K].
__global__ void __launch_bounds__(256)
fp8_quant_transpose_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q_t, long long ldq,
                           float* __restrict__ s, int T, int K, bool ue8m0) {
  __shared__ __align__(16) uint32_t tile[128 * 32];
  __shared__ float red[8][64];
  __shared__ __align__(16) uint8_t outb[64 * 128];
  const int t0 = blockIdx.y * 128, k0 = blockIdx.x * 64;
  const int tid = threadIdx.x;
  for (int i = tid; i < 1024; i += 256) {
    const int r = i >> 3, seg = i & 7;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (t0 + r < T) v = *reinterpret_cast<const uint4*>(x + static_cast<long long>(t0 + r) * ldx + k0 + seg * 8);
    *reinterpret_cast<uint4*>(tile + r * 32 + seg * 4) = v;
  }
  __syncthreads();
  const int pair = tid & 31, part = tid >> 5;
  float f0[16], f1[16];
  float a0 = 0.f, a1 = 0.f;
  #pragma unroll
  for (int j = 0; j < 16; ++j) {
    const uint32_t w = tile[(part * 16 + j) * 32 + pair];
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
    f0[j] = f.x; f1[j] = f.y;
    a0 = fmaxf(a0, fabsf(f.x)); a1 = fmaxf(a1, fabsf(f.y));
  }
  red[part][2 * pair] = a0;
  red[part][2 * pair + 1] = a1;
  __syncthreads();
  float m0 = 0.f, m1 = 0.f;
  #pragma unroll
  for (int p8 = 0; p8 < 8; ++p8) { m0 = fmaxf(m0, red[p8][2 * pair]); m1 = fmaxf(m1, red[p8][2 * pair + 1]); }
  const float s0 = fp8_block_scale(m0, ue8m0), s1 = fp8_block_scale(m1, ue8m0);
  if (part == 0)
    *reinterpret_cast<float2*>(s + static_cast<long long>(blockIdx.y) * K + k0 + 2 * pair) = make_float2(s0, s1);
  const float i0 = 1.f / s0, i1 = 1.f / s1;
  uint4 o0, o1;
  o0.x = quant4_e4m3(f0[0], f0[1], f0[2], f0[3], i0);    o0.y = quant4_e4m3(f0[4], f0[5], f0[6], f0[7], i0);
  o0.z = quant4_e4m3(f0[8], f0[9], f0[10], f0[11], i0);  o0.w = quant4_e4m3(f0[12], f0[13], f0[14], f0[15], i0);
  o1.x = quant4_e4m3(f1[0], f1[1], f1[2], f1[3], i1);    o1.y = quant4_e4m3(f1[4], f1[5], f1[6], f1[7], i1);
  o1.z = quant4_e4m3(f1[8], f1[9], f1[10], f1[11], i1);  o1.w = quant4_e4m3(f1[12], f1[13], f1[14], f1[15], i1);
  const int chunk = part ^ (pair & 7);
  *reinterpret_cast<uint4*>(outb + (2 * pair) * 128 + chunk * 16) = o0;
  *reinterpret_cast<uint4*>(outb + (2 * pair + 1) * 128 + chunk * 16) = o1;
  __syncthreads();
  for (int i = tid; i < 512; i += 256) {
    const int ch = i >> 3, seg = i & 7;
    const uint4 v = *reinterpret_cast<const uint4*>(outb + ch * 128 + (seg ^ ((ch >> 1) & 7)) * 16);
    *reinterpret_cast<uint4*>(q_t + static_cast<long long>(k0 + ch) * ldq + t0 + seg * 16) = v;
  }
}

static const __nv_bfloat16* bfc(const at::Tensor& t) { return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr()); }
static __nv_bfloat16* bfm(at::Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }

static void check_gu(const at::Tensor& gu, const char* who) {
  TORCH_CHECK(gu.is_cuda() && gu.scalar_type() == at::kBFloat16 && gu.dim() == 2 && gu.stride(1) == 1 && gu.size(1) % 256 == 0 &&
              gu.stride(0) % 4 == 0 && (reinterpret_cast<uintptr_t>(gu.data_ptr()) & 7) == 0,
              who, ": bf16 [R, 2I] with I a multiple of 128");
}
static const float* prob_ptr(const c10::optional<at::Tensor>& prob, int64_t R, const char* who) {
  if (!prob.has_value()) return nullptr;
  TORCH_CHECK(prob->is_cuda() && prob->scalar_type() == at::kFloat && prob->is_contiguous() && prob->numel() == R, who,
              ": prob must be fp32 [R]");
  return prob->data_ptr<float>();
}

// (q [R, I] e4m3, s_t [I/128, R] fp32, act [R, I] bf16 or empty)
std::tuple<at::Tensor, at::Tensor, at::Tensor> swiglu_quant_fwd(const at::Tensor& gu, const c10::optional<at::Tensor>& prob,
                                                                bool ue8m0, bool want_act) {
  check_gu(gu, "swiglu_quant_fwd");
  const c10::cuda::CUDAGuard guard(gu.device());
  const int64_t R = gu.size(0), I = gu.size(1) / 2;
  const float* pp = prob_ptr(prob, R, "swiglu_quant_fwd");
  at::Tensor q = at::empty({R, I}, gu.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor s_t = at::empty({I / 128, R}, gu.options().dtype(at::kFloat));
  at::Tensor act = at::empty({want_act ? R : 0, I}, gu.options());
  if (R == 0) return {q, s_t, act};
  const int64_t units = R * (I / 128);
  const int blocks = static_cast<int>(std::min<int64_t>((units * 32 + 255) / 256, 148 * 16));
  swiglu_quant_fwd_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      bfc(gu), gu.stride(0), pp, reinterpret_cast<uint8_t*>(q.data_ptr()), s_t.data_ptr<float>(), want_act ? bfm(act) : nullptr, R,
      static_cast<int>(I), ue8m0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {q, s_t, act};
}

// (dgu [R, 2I] bf16, gq [R, 2I] e4m3, gs_t [2I/128, R] fp32, act [R, I] bf16 or empty, dprob_part [I/128, R] fp32 or empty)
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> swiglu_quant_bwd(
    const at::Tensor& dact, const at::Tensor& gu, const c10::optional<at::Tensor>& prob, bool ue8m0, bool want_act) {
  check_gu(gu, "swiglu_quant_bwd");
  const c10::cuda::CUDAGuard guard(gu.device());
  const int64_t R = gu.size(0), I = gu.size(1) / 2;
  TORCH_CHECK(dact.is_cuda() && dact.scalar_type() == at::kBFloat16 && dact.is_contiguous() && dact.dim() == 2 && dact.size(0) == R &&
              dact.size(1) == I, "swiglu_quant_bwd: dact must be contiguous bf16 [R, I]");
  const float* pp = prob_ptr(prob, R, "swiglu_quant_bwd");
  at::Tensor dgu = at::empty({R, 2 * I}, gu.options());
  at::Tensor gq = at::empty({R, 2 * I}, gu.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor gs_t = at::empty({2 * I / 128, R}, gu.options().dtype(at::kFloat));
  at::Tensor act = at::empty({want_act ? R : 0, I}, gu.options());
  at::Tensor dpp = at::empty({pp ? I / 128 : 0, R}, gu.options().dtype(at::kFloat));
  if (R == 0) return {dgu, gq, gs_t, act, dpp};
  const int64_t units = R * (I / 128);
  const int blocks = static_cast<int>(std::min<int64_t>((units * 32 + 255) / 256, 148 * 16));
  swiglu_quant_bwd_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      bfc(dact), bfc(gu), gu.stride(0), pp, bfm(dgu), reinterpret_cast<uint8_t*>(gq.data_ptr()), gs_t.data_ptr<float>(),
      want_act ? bfm(act) : nullptr, pp ? dpp.data_ptr<float>() : nullptr, R, static_cast<int>(I), ue8m0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dgu, gq, gs_t, act, dpp};
}

// (q_t [K, ceil(T/128)*128] e4m3, s [ceil(T/128), K] fp32)
std::tuple<at::Tensor, at::Tensor> fp8_quant_transpose(const at::Tensor& x, bool ue8m0) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "fp8_quant_transpose: bf16 [T, K]");
  const int64_t T = x.size(0), K = x.size(1);
  TORCH_CHECK(K % 64 == 0 && x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0,
              "fp8_quant_transpose: K must be a multiple of 64 and rows 16-byte aligned");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t tb = (T + 127) / 128;
  at::Tensor q_t = at::empty({K, tb * 128}, x.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor s = at::empty({tb, K}, x.options().dtype(at::kFloat));
  if (T == 0) return {q_t, s};
  dim3 grid(static_cast<unsigned>(K / 64), static_cast<unsigned>(tb));
  fp8_quant_transpose_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      bfc(x), x.stride(0), reinterpret_cast<uint8_t*>(q_t.data_ptr()), tb * 128, s.data_ptr<float>(), static_cast<int>(T),
      static_cast<int>(K), ue8m0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {q_t, s};
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("swiglu_quant_fwd(Tensor gu, Tensor? prob, bool ue8m0, bool want_act) -> (Tensor, Tensor, Tensor)", &pfb::swiglu_quant_fwd);
  m.def("swiglu_quant_bwd(Tensor dact, Tensor gu, Tensor? prob, bool ue8m0, bool want_act) -> (Tensor, Tensor, Tensor, Tensor, Tensor)",
        &pfb::swiglu_quant_bwd);
  m.def("fp8_quant_transpose(Tensor x, bool ue8m0) -> (Tensor, Tensor)", &pfb::fp8_quant_transpose);
}
