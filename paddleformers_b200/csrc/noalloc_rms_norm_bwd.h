// RMSNorm backward for callers that cannot allocate device memory. This entry point has no counterpart in the
// reference: it exists only in this library.
//
// Who needs it: code that calls the kernels directly from C or C++ (no torch caching allocator behind it) at a moment
// when cudaMalloc is not an option - a process that has deliberately filled HBM with its model state so that any
// further allocation would fail, or a latency-critical section where the device-wide synchronisation that
// cudaMalloc / cudaFree imply is unacceptable. The regular entry point (torch.ops.pfb200.rms_norm_bwd) takes its
// weight-gradient scratch from the caller or from torch; this one keeps that scratch inside the library.
//
// The scratch (per-block partial sums of the weight gradient) is a file-scope `static __device__` array of
// PFB_NOALLOC_PARTIAL_ROWS x PFB_NOALLOC_MAX_H floats = 2 MiB. Every GPU on which the library is loaded holds it
// until the process exits.
//
// Rules for callers:
//  * H must be a multiple of 8 and at most PFB_NOALLOC_MAX_H; larger rows are rejected with an error message.
//  * All pointers are device pointers of the current device, 16-byte aligned; dy rows may be strided
//    (dy_row_stride in elements, multiple of 8), x / dres / dx are contiguous [T, H].
//  * The first call on each device looks up the device address of the scratch array (cudaGetSymbolAddress) and caches
//    it; make that first call before starting any stream capture on that device.
//  * All calls on one device share the one scratch array, and it keeps the previous call's contents. Nothing in it
//    has to start at zero (every launch overwrites the part it later reads), but two calls whose kernels overlap on
//    the GPU - different streams, no ordering between them - race on it. Serialise them.
//  * The call enqueues two kernels on `stream` and returns; it never synchronises and never allocates.
#pragma once

#define PFB_NOALLOC_MAX_H 8192
#define PFB_NOALLOC_PARTIAL_ROWS 64

#ifdef __cplusplus
extern "C" {
#endif

// dx[T,H] (bf16) = d(rmsnorm)/dx applied to dy (+ dres when not null); dw[H] (fp32) = or += sum_t dy * x * rstd.
//   dy, x, w, dres, dx: bf16; rstd: fp32 [T]; dw: fp32 [H]; accumulate != 0 adds to the existing dw.
// Returns 0 on success. On failure returns a negative code and, when err != NULL, writes a NUL-terminated message of
// at most err_len bytes: -1 invalid argument (including H beyond the maximum), -2 CUDA error.
int pfb_rms_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                             void* dx, float* dw, int T, int H, long long dy_row_stride, int accumulate,
                             void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
