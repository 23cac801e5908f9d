// Host launchers and torch bindings of the tensor-core-scaled fp8 GEMM (gemm_mxf8_sm100.cuh).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "gemm_mxf8_sm100.cuh"
#include "status.h"
#include "tma_host.h"

namespace pfb {

template <int BN, int STAGES, bool GROUPED>
static void launch_mx(const CUtensorMap& tmA, const CUtensorMap& tmB, const MxGemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm_mxf8_kernel<BN, STAGES, GROUPED>;
  constexpr int smem = MxSmem<BN, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<grid, MX_THREADS, smem, stream>>>(tmA, tmB, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <int BN, int STAGES>
static void dispatch_mx(bool grouped, const CUtensorMap& tmA, const CUtensorMap& tmB, const MxGemmParams& p, int grid,
                        cudaStream_t stream) {
  if (grouped) launch_mx<BN, STAGES, true>(tmA, tmB, p, grid, stream);
  else launch_mx<BN, STAGES, false>(tmA, tmB, p, grid, stream);
}

static bool is_fp8(const at::Tensor& t) { return t.scalar_type() == at::kFloat8_e4m3fn || t.scalar_type() == at::kByte; }

// Tile width for an output of n columns per matrix: the candidate with the least padded work, wider tiles first on a tie.
int64_t mxf8_tile_n(int64_t n) {
  const int cands[3] = {240, 192, 128};
  int best = 240;
  int64_t best_cost = INT64_MAX;
  for (int bn : cands) {
    const int64_t padded = (n + bn - 1) / bn * bn;
    // narrower tiles re-read the A operand more often: charge them a few per cent
    const int64_t cost = padded * (bn == 240 ? 100 : bn == 192 ? 104 : 112);
    if (cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

// aq: [M, K] e4m3; sfa: packed exponents of aq for 128-row tiles; bq: [N, K] e4m3 (grouped: [E*N, K]);
// sfb: packed exponents of bq for bn-row tiles; out: [M, N] bf16, or fp32 that the product is added to.
void gemm_mxf8(const at::Tensor& aq, const at::Tensor& sfa, const at::Tensor& bq, const at::Tensor& sfb, at::Tensor& out,
               const c10::optional<at::Tensor>& block_expert, int64_t n_per_expert, int64_t bn) {
  TORCH_CHECK(aq.is_cuda() && bq.is_cuda() && out.is_cuda() && is_fp8(aq) && is_fp8(bq), "gemm_mxf8: CUDA e4m3 operands");
  TORCH_CHECK(aq.dim() == 2 && bq.dim() == 2 && aq.is_contiguous() && bq.is_contiguous(), "gemm_mxf8: contiguous 2-D operands");
  TORCH_CHECK(bn == 128 || bn == 192 || bn == 240, "gemm_mxf8: tile width must be 128, 192 or 240");
  const c10::cuda::CUDAGuard guard(aq.device());
  const bool grouped = block_expert.has_value();
  const int M = aq.size(0), K = aq.size(1);
  const int rows_b = bq.size(0);
  const int N = grouped ? static_cast<int>(n_per_expert) : rows_b;
  TORCH_CHECK(bq.size(1) == K && K % MX_BK == 0, "gemm_mxf8: K must match and be a multiple of 128");
  const int kbs = K / MX_BK, kgs = (kbs + 3) / 4;
  const int m_blocks = (M + MX_BM - 1) / MX_BM, n_blocks = (N + bn - 1) / static_cast<int>(bn);
  const int groups = grouped ? rows_b / std::max(N, 1) : 1;
  const int sfb_rows = (static_cast<int>(bn) + 127) / 128 * 128;
  TORCH_CHECK(!grouped || (N > 0 && rows_b % N == 0), "grouped gemm_mxf8: stacked [E * N, K] weights");
  TORCH_CHECK(sfa.scalar_type() == at::kInt && sfa.is_contiguous() && sfa.numel() == static_cast<int64_t>(m_blocks) * kgs * 128,
              "gemm_mxf8: sfa must hold [ceil(M/128), ceil(K/512), 128] packed exponent words");
  TORCH_CHECK(sfb.scalar_type() == at::kInt && sfb.is_contiguous() &&
              sfb.numel() == static_cast<int64_t>(groups) * n_blocks * kgs * sfb_rows,
              "gemm_mxf8: sfb must hold [E * ceil(N/bn), ceil(K/512), ceil(bn/128)*128] packed exponent words");
  const bool acc = out.scalar_type() == at::kFloat;
  TORCH_CHECK((acc || out.scalar_type() == at::kBFloat16) && out.dim() == 2 && out.size(0) == M && out.size(1) == N &&
              out.stride(1) == 1 && out.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0,
              "gemm_mxf8: out must be bf16 or fp32 [M, N]");
  if (grouped)
    TORCH_CHECK(block_expert->scalar_type() == at::kInt && block_expert->is_cuda() && block_expert->numel() * MX_BM >= M);
  if (M == 0 || N == 0) return;
  MxGemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.D = acc ? nullptr : reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.Dacc = acc ? out.data_ptr<float>() : nullptr;
  p.ldd = out.stride(0);
  p.sfa = reinterpret_cast<const uint32_t*>(sfa.data_ptr());
  p.sfb = reinterpret_cast<const uint32_t*>(sfb.data_ptr());
  p.m_blocks = m_blocks; p.n_blocks = n_blocks; p.k_blocks = kbs; p.k_groups = kgs;
  p.group_m = 8;
  p.block_expert = grouped ? block_expert->data_ptr<int>() : nullptr;
  p.n_per_expert = static_cast<int>(n_per_expert);
  p.status = status_word();
  const CUtensorMap tmA = make_tma_2d(aq.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, MX_BM, MX_BK);
  const CUtensorMap tmB = make_tma_2d(bq.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows_b, K, K, static_cast<uint32_t>(bn), MX_BK);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int grid = std::min(m_blocks * n_blocks, sms);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (bn == 240) dispatch_mx<240, 4>(grouped, tmA, tmB, p, grid, stream);
  else if (bn == 192) dispatch_mx<192, 5>(grouped, tmA, tmB, p, grid, stream);
  else dispatch_mx<128, 6>(grouped, tmA, tmB, p, grid, stream);
  count_launch();
}

// Packed exponent words of a scale tensor for tiles of `bt` rows (see mx_pack_scales_kernel). transposed = true: scales
// [K/128, rows] of a 1x128-quantised activation; false: [rows/128, K/128] of a 128x128-quantised weight.
at::Tensor mx_pack_scales(const at::Tensor& s, bool transposed, int64_t rows_per_group, int64_t groups, int64_t bt) {
  TORCH_CHECK(s.is_cuda() && s.scalar_type() == at::kFloat && s.dim() == 2 && s.stride(1) == 1, "mx_pack_scales: fp32 2-D scales");
  TORCH_CHECK(bt >= 8 && bt <= 256 && rows_per_group > 0 && groups > 0, "mx_pack_scales: tile rows in [8, 256]");
  const c10::cuda::CUDAGuard guard(s.device());
  const int64_t rows = rows_per_group * groups;
  const int64_t kbs = transposed ? s.size(0) : s.size(1);
  TORCH_CHECK(transposed ? s.size(1) >= rows : s.size(0) * 128 >= rows, "mx_pack_scales: the scales must cover every row");
  const int64_t kgs = (kbs + 3) / 4, tiles = (rows_per_group + bt - 1) / bt, sfr = (bt + 127) / 128 * 128;
  at::Tensor out = at::empty({groups * tiles, kgs, sfr}, s.options().dtype(at::kInt));
  const int64_t total = out.numel();
  if (total == 0) return out;
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 8));
  mx_pack_scales_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      s.data_ptr<float>(), s.stride(0), transposed ? 0 : 1, reinterpret_cast<uint32_t*>(out.data_ptr()),
      static_cast<int>(rows_per_group), static_cast<int>(groups), static_cast<int>(bt), static_cast<int>(kbs), status_word());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("gemm_mxf8(Tensor aq, Tensor sfa, Tensor bq, Tensor sfb, Tensor(a!) out, Tensor? block_expert, int n_per_expert, int bn) -> ()",
        &pfb::gemm_mxf8);
  m.def("mx_pack_scales(Tensor s, bool transposed, int rows_per_group, int groups, int bt) -> Tensor", &pfb::mx_pack_scales);
  m.def("mxf8_tile_n(int n) -> int", &pfb::mxf8_tile_n);
}
