// Host launchers and torch bindings of the block-scaled fp8 GEMM and its quantisation kernels (gemm_fp8_sm100.cuh).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "gemm_fp8_sm100.cuh"
#include "status.h"
#include "tma_host.h"

namespace pfb {

constexpr int F8_STAGES = 6;

template <bool GROUPED>
static void launch_fp8(const CUtensorMap& tmA, const CUtensorMap& tmB, const Fp8GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm_fp8_blockscaled_kernel<F8_STAGES, GROUPED>;
  constexpr int smem = Fp8Smem<F8_STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<grid, F8_THREADS, smem, stream>>>(tmA, tmB, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

static bool is_fp8(const at::Tensor& t) { return t.scalar_type() == at::kFloat8_e4m3fn || t.scalar_type() == at::kByte; }

// aq: [M, K] e4m3; sa_t: [K/128, M] fp32; bq: [N, K] e4m3 (grouped: [E*N, K]); sb: [rows(bq)/128, K/128] fp32; out: [M, N] bf16
void gemm_fp8(const at::Tensor& aq, const at::Tensor& sa_t, const at::Tensor& bq, const at::Tensor& sb, at::Tensor& out,
              const c10::optional<at::Tensor>& block_expert, int64_t n_per_expert) {
  TORCH_CHECK(aq.is_cuda() && bq.is_cuda() && out.is_cuda() && is_fp8(aq) && is_fp8(bq), "gemm_fp8: CUDA e4m3 operands");
  TORCH_CHECK(aq.dim() == 2 && bq.dim() == 2 && aq.is_contiguous() && bq.is_contiguous(), "gemm_fp8: contiguous 2-D operands");
  const c10::cuda::CUDAGuard guard(aq.device());
  const bool grouped = block_expert.has_value();
  const int M = aq.size(0), K = aq.size(1);
  const int rows_b = bq.size(0);
  const int N = grouped ? static_cast<int>(n_per_expert) : rows_b;
  TORCH_CHECK(bq.size(1) == K && K % F8_BK == 0, "gemm_fp8: K must match and be a multiple of 128");
  const int kbs = K / F8_BK;
  TORCH_CHECK(sa_t.scalar_type() == at::kFloat && sa_t.dim() == 2 && sa_t.size(0) == kbs && sa_t.size(1) >= M && sa_t.stride(1) == 1,
              "gemm_fp8: sa_t must be fp32 [K/128, M]");
  TORCH_CHECK(sb.scalar_type() == at::kFloat && sb.is_contiguous() && sb.dim() == 2 && sb.size(1) == kbs &&
              sb.size(0) == (rows_b + F8_BN - 1) / F8_BN, "gemm_fp8: sb must be fp32 [ceil(rows/128), K/128]");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.stride(1) == 1 &&
              out.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0, "gemm_fp8: bf16 out [M, N]");
  if (grouped) {
    TORCH_CHECK(N % F8_BN == 0 && rows_b % N == 0, "grouped gemm_fp8: n_per_expert % 128 == 0 and stacked rows");
    TORCH_CHECK(block_expert->scalar_type() == at::kInt && block_expert->is_cuda() && block_expert->numel() * F8_BM >= M);
  }
  if (M == 0 || N == 0) return;
  Fp8GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.D = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.ldd = out.stride(0);
  p.sa_t = sa_t.data_ptr<float>(); p.sa_ld = sa_t.stride(0);
  p.sb = sb.data_ptr<float>();
  p.m_blocks = (M + F8_BM - 1) / F8_BM;
  p.n_blocks = (N + F8_BN - 1) / F8_BN;
  p.k_blocks = kbs;
  p.group_m = 8;
  p.block_expert = grouped ? block_expert->data_ptr<int>() : nullptr;
  p.n_per_expert = static_cast<int>(n_per_expert);
  p.status = status_word();
  const CUtensorMap tmA = make_tma_2d(aq.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, F8_BM, F8_BK);
  const CUtensorMap tmB = make_tma_2d(bq.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows_b, K, K, F8_BN, F8_BK);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int grid = std::min(p.m_blocks * p.n_blocks, sms);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (grouped) launch_fp8<true>(tmA, tmB, p, grid, stream);
  else launch_fp8<false>(tmA, tmB, p, grid, stream);
  count_launch();
}

std::tuple<at::Tensor, at::Tensor> fp8_quant_act(const at::Tensor& x, bool ue8m0) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "fp8_quant_act: bf16 [T, K]");
  const int64_t T = x.size(0), K = x.size(1);
  TORCH_CHECK(K % 128 == 0 && x.stride(0) % 4 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 7) == 0,
              "fp8_quant_act: K must be a multiple of 128");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor q = at::empty({T, K}, x.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor s_t = at::empty({K / 128, T}, x.options().dtype(at::kFloat));
  if (T == 0) return {q, s_t};
  const int64_t units = T * (K / 128);
  const int blocks = static_cast<int>(std::min<int64_t>((units * 32 + 255) / 256, 148 * 16));
  fp8_quant_act_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), x.stride(0), reinterpret_cast<uint8_t*>(q.data_ptr()),
      s_t.data_ptr<float>(), static_cast<int>(T), static_cast<int>(K), ue8m0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {q, s_t};
}

std::tuple<at::Tensor, at::Tensor> fp8_quant_weight(const at::Tensor& w, bool ue8m0) {
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1, "fp8_quant_weight: bf16 [N, K]");
  const int64_t N = w.size(0), K = w.size(1);
  TORCH_CHECK(K % 128 == 0 && w.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(w.data_ptr()) & 15) == 0,
              "fp8_quant_weight: K must be a multiple of 128");
  const c10::cuda::CUDAGuard guard(w.device());
  at::Tensor q = at::empty({N, K}, w.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor s = at::empty({(N + 127) / 128, K / 128}, w.options().dtype(at::kFloat));
  if (N == 0) return {q, s};
  dim3 grid(static_cast<unsigned>(K / 128), static_cast<unsigned>((N + 127) / 128));
  fp8_quant_weight_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(w.data_ptr()), w.stride(0), reinterpret_cast<uint8_t*>(q.data_ptr()), s.data_ptr<float>(),
      static_cast<int>(N), static_cast<int>(K), ue8m0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {q, s};
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("gemm_fp8(Tensor aq, Tensor sa_t, Tensor bq, Tensor sb, Tensor(a!) out, Tensor? block_expert, int n_per_expert) -> ()",
        &pfb::gemm_fp8);
  m.def("fp8_quant_act(Tensor x, bool ue8m0) -> (Tensor, Tensor)", &pfb::fp8_quant_act);
  m.def("fp8_quant_weight(Tensor w, bool ue8m0) -> (Tensor, Tensor)", &pfb::fp8_quant_weight);
}
