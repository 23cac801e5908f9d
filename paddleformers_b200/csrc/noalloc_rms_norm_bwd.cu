// Implementation of pfb_rms_norm_bwd_noalloc (see noalloc_rms_norm_bwd.h): a variant of the RMSNorm backward kernel
// whose weight-gradient partial sums live in a static device array instead of caller-provided scratch.
// Nothing in this file allocates: no cudaMalloc / cudaFree, no torch, no library routine that allocates.
#include "noalloc_rms_norm_bwd.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

namespace {

// Shared by every call on this device; keeps the last call's partial sums. Host code must not pass this name to a
// kernel: on the host it is only a handle for cudaGetSymbolAddress.
static __device__ __align__(256) float g_dw_partials[PFB_NOALLOC_PARTIAL_ROWS * PFB_NOALLOC_MAX_H];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ float warp_sum(float v) {
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  return warp_sum(l < nw ? red[l] : 0.f);
}

// Block b handles rows b, b + gridDim.x, ...: writes dx for them and its partial weight gradient to
// partials[b, 0..H). Every block writes all H columns of its row, so no entry that the reduction reads is stale.
template <int PER_THREAD>
__global__ void rms_norm_bwd_static_scratch_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                                   float* __restrict__ partials, int T, int H, long long dy_stride) {
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
        const bf16x8 a = dyr[i], b = xr[i], ww = wr[i];
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __bfloat1622float2(a.v[j]), fb = __bfloat1622float2(b.v[j]), fw = __bfloat1622float2(ww.v[j]);
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
          if (drr) { const float2 fr = __bfloat1622float2(r.v[j]); a0 += fr.x; a1 += fr.y; }
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
      float4* dst = reinterpret_cast<float4*>(partials + static_cast<long long>(blockIdx.x) * H + i * 8);
      dst[0] = make_float4(dwacc[c][0], dwacc[c][1], dwacc[c][2], dwacc[c][3]);
      dst[1] = make_float4(dwacc[c][4], dwacc[c][5], dwacc[c][6], dwacc[c][7]);
    }
  }
}

__global__ void rms_norm_dw_fold_kernel(const float* __restrict__ partials, float* __restrict__ dw, int P, int H,
                                        int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partials[static_cast<long long>(p) * H + h];
  dw[h] = accumulate ? dw[h] + s : s;
}

int fail(int code, char* err, int err_len, const char* msg, const char* detail = nullptr) {
  if (err && err_len > 0) {
    if (detail) snprintf(err, err_len, "%s: %s", msg, detail);
    else snprintf(err, err_len, "%s", msg);
  }
  return code;
}

// Device address of the static scratch array for the current device; looked up once per device.
int scratch_for_current_device(float** out, char* err, int err_len) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(-2, err, err_len, "cudaGetDevice failed", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(-1, err, err_len, "device index out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_dw_partials);
    if (e != cudaSuccess || p == nullptr)
      return fail(-2, err, err_len, "cudaGetSymbolAddress(g_dw_partials) failed", cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int pfb_rms_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                        void* dx, float* dw, int T, int H, long long dy_row_stride, int accumulate,
                                        void* stream, char* err, int err_len) {
  if (!dy || !x || !w || !rstd || !dx || !dw) return fail(-1, err, err_len, "null pointer argument");
  if (T < 0 || H <= 0) return fail(-1, err, err_len, "T must be >= 0 and H > 0");
  if (H % 8 != 0) return fail(-1, err, err_len, "H must be a multiple of 8");
  if (H > PFB_NOALLOC_MAX_H) {
    char msg[160];
    snprintf(msg, sizeof(msg), "H = %d exceeds the built-in scratch (maximum %d columns); use the regular entry point "
             "with caller-provided scratch", H, PFB_NOALLOC_MAX_H);
    return fail(-1, err, err_len, msg);
  }
  if (dy_row_stride < H || dy_row_stride % 8 != 0) return fail(-1, err, err_len, "dy_row_stride must be >= H and a multiple of 8");
  if (!aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx) || !aligned16(dw) || (dres && !aligned16(dres)))
    return fail(-1, err, err_len, "pointers must be 16-byte aligned");
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch, err, err_len);
  if (rc != 0) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int P = T < PFB_NOALLOC_PARTIAL_ROWS ? (T > 0 ? T : 1) : PFB_NOALLOC_PARTIAL_ROWS;
  const auto* dyb = static_cast<const __nv_bfloat16*>(dy);
  const auto* xb = static_cast<const __nv_bfloat16*>(x);
  const auto* wb = static_cast<const __nv_bfloat16*>(w);
  const auto* drb = static_cast<const __nv_bfloat16*>(dres);
  auto* dxb = static_cast<__nv_bfloat16*>(dx);
  constexpr int threads = 256;
  const int per = (H / 8 + threads - 1) / threads;
  if (T > 0) {
    if (per <= 1) rms_norm_bwd_static_scratch_kernel<1><<<P, threads, 0, s>>>(dyb, xb, wb, rstd, drb, dxb, scratch, T, H, dy_row_stride);
    else if (per <= 2) rms_norm_bwd_static_scratch_kernel<2><<<P, threads, 0, s>>>(dyb, xb, wb, rstd, drb, dxb, scratch, T, H, dy_row_stride);
    else rms_norm_bwd_static_scratch_kernel<4><<<P, threads, 0, s>>>(dyb, xb, wb, rstd, drb, dxb, scratch, T, H, dy_row_stride);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(-2, err, err_len, "launch of the backward kernel failed", cudaGetErrorString(e));
  }
  // With T == 0 no partials were written: fold zero rows so that dw is zeroed (or left unchanged when accumulating).
  rms_norm_dw_fold_kernel<<<(H + 255) / 256, 256, 0, s>>>(scratch, dw, T > 0 ? P : 0, H, accumulate ? 1 : 0);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(-2, err, err_len, "launch of the fold kernel failed", cudaGetErrorString(e));
  return 0;
}
