// Host launchers and torch bindings of the fused all-gather-GEMM / GEMM-reduce-scatter kernels (gemm_comm_sm100.cuh).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "gemm_comm_sm100.cuh"
#include "status.h"
#include "tma_host.h"

#include <cstdlib>

namespace pfb {

template <int BN, int STAGES, bool B_MN, int EPI, int MODE>
static void launch_comm(const CUtensorMap& tmA, const CUtensorMap& tmB, const StageMaps& sm, const GemmParams& p,
                        const CommParams& c, int grid, cudaStream_t stream) {
  auto kern = gemm_comm_kernel<BN, STAGES, B_MN, EPI, MODE>;
  constexpr int smem = GemmSmem<BN, STAGES>::TOTAL + (MODE == MODE_RS ? RS_STAGING_BYTES : 0);
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, smem, stream>>>(tmA, tmB, sm, p, c);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <int MODE>
static void dispatch_comm(int BN, bool b_mn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const StageMaps& sm,
                          const GemmParams& p, const CommParams& c, int grid, cudaStream_t s) {
#define PFB_C(BNV, ST, BMN, E)                                                                  \
  if (BN == BNV && b_mn == BMN && epi == E) { launch_comm<BNV, ST, BMN, E, MODE>(tmA, tmB, sm, p, c, grid, s); return; }
  PFB_C(256, 4, false, EPI_STORE_BF16)
  PFB_C(256, 4, true, EPI_STORE_BF16)
  PFB_C(128, 6, false, EPI_STORE_BF16)
  PFB_C(128, 6, true, EPI_STORE_BF16)
  if constexpr (MODE == MODE_AG) {
    PFB_C(256, 4, false, EPI_SWIGLU_BF16)
    PFB_C(128, 6, false, EPI_SWIGLU_BF16)
  }
#undef PFB_C
  TORCH_CHECK(false, "fused comm GEMM: unsupported combination");
}

static int sms() {
  static int n = 0;
  if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

static int pick_bn(int M, int N, bool swiglu, int ctas) {
  auto cost = [&](int bn) {
    int nn = swiglu ? (N / 2 + bn / 2 - 1) / (bn / 2) : (N + bn - 1) / bn;
    long long tiles = static_cast<long long>((M + GEMM_BM - 1) / GEMM_BM) * nn;
    return ((tiles + ctas - 1) / ctas) * bn;
  };
  return cost(128) * 3 < cost(256) * 2 ? 128 : 256;   // 256-wide tiles measured 1.4-1.5x the rate of 128-wide ones
}

// out[T, N] (SwiGLU: [T, N/2]) = gather(G)[T, K] @ B^T with B = weight [N, K] or (b_mn) [K, N]. G is this rank's
// symmetric gathered buffer whose own slice (rows rank*R .. +R) has already been written on the current stream.
void ag_gemm(const at::Tensor& G, const at::Tensor& peer_G_ptrs, const at::Tensor& weight, at::Tensor& out,
             const c10::optional<at::Tensor>& out2, int64_t epi, bool b_mn, int64_t ready_ptr,
             const at::Tensor& peer_ready_ptrs, at::Tensor& blk_flags, const at::Tensor& epoch, int64_t rank, int64_t tp, int64_t n_copy) {
  TORCH_CHECK(G.is_cuda() && G.dim() == 2 && G.is_contiguous() && G.scalar_type() == at::kBFloat16);
  TORCH_CHECK(weight.scalar_type() == at::kBFloat16 && weight.dim() == 2 && weight.stride(1) == 1);
  TORCH_CHECK(tp >= 2 && tp <= COMM_MAX_RANKS && peer_G_ptrs.numel() == tp && peer_ready_ptrs.numel() == tp);
  TORCH_CHECK(!peer_G_ptrs.is_cuda() && !peer_ready_ptrs.is_cuda() && peer_G_ptrs.scalar_type() == at::kLong);
  const c10::cuda::CUDAGuard guard(G.device());
  const int T = G.size(0), K = G.size(1);
  TORCH_CHECK(T % (tp * GEMM_BM) == 0, "ag_gemm: tokens must be a multiple of tp * 128");
  TORCH_CHECK(K % 128 == 0, "ag_gemm: K must be a multiple of 128");
  const int Kb = b_mn ? weight.size(0) : weight.size(1);
  const int N = b_mn ? weight.size(1) : weight.size(0);
  TORCH_CHECK(K == Kb);
  const bool swiglu = epi == EPI_SWIGLU_BF16;
  TORCH_CHECK(epi == EPI_STORE_BF16 || swiglu);
  TORCH_CHECK(out.size(0) == T && out.size(1) == (swiglu ? N / 2 : N) && out.stride(1) == 1 && out.scalar_type() == at::kBFloat16);
  TORCH_CHECK(blk_flags.scalar_type() == at::kInt && blk_flags.numel() >= T / GEMM_BM && blk_flags.is_cuda());
  const int ncopy = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(n_copy, 32)));
  const int gemm_ctas = sms() - ncopy;
  const int BN = pick_bn(T, N, swiglu, gemm_ctas);
  GemmParams p;
  p.M = T; p.N = N; p.K = K;
  p.D = out.data_ptr(); p.ldd = out.stride(0);
  p.D2 = nullptr; p.ldd2 = 0;
  if (out2.has_value()) { p.D2 = out2->data_ptr(); p.ldd2 = out2->stride(0); }
  p.m_blocks = T / GEMM_BM;
  p.n_blocks = swiglu ? (N / 2 + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
  p.k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.group_m = 4;
  p.block_expert = nullptr; p.n_per_expert = 0; p.expert_rows = nullptr; p.tiles_per_expert = 0; p.d_expert_stride = 0;
  p.status = status_word();
  CommParams c{};
  c.mode = MODE_AG; c.rank = rank; c.tp = tp; c.rows_per_rank = T / tp; c.epoch_ptr = epoch.data_ptr<int>(); c.n_copy_ctas = ncopy;
  for (int q = 0; q < tp; ++q) {
    c.peer_G[q] = reinterpret_cast<const __nv_bfloat16*>(peer_G_ptrs.data_ptr<int64_t>()[q]);
    c.peer_ready[q] = reinterpret_cast<int*>(peer_ready_ptrs.data_ptr<int64_t>()[q]);
  }
  c.G = reinterpret_cast<__nv_bfloat16*>(G.data_ptr());
  c.ready = reinterpret_cast<int*>(ready_ptr);
  c.blk_flags = blk_flags.data_ptr<int>();
  c.row_bytes = static_cast<long long>(K) * 2;
  const uint32_t b_box_rows = swiglu ? BN / 2 : BN;
  CUtensorMap tmA = make_tma_2d(G.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, K, GEMM_BM, 64);
  CUtensorMap tmB = b_mn ? make_tma_2d(weight.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, weight.stride(0), GEMM_BK, 64)
                         : make_tma_2d(weight.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, weight.stride(0), b_box_rows, 64);
  const int tiles = p.m_blocks * p.n_blocks;
  const int grid = ncopy + std::min(tiles, gemm_ctas);
  StageMaps sm{};
  for (int q = 0; q < COMM_MAX_RANKS; ++q) sm.m[q] = tmA;  // unused in this mode
  dispatch_comm<MODE_AG>(BN, b_mn, static_cast<int>(epi), tmA, tmB, sm, p, c, grid, at::cuda::getCurrentCUDAStream());
  count_launch();
}

// out[T/tp, N] = reduce_scatter_rows(x[T, K] @ B^T) over the tp ranks; B = weight [N, K] or (b_mn) [K, N].
void gemm_rs(const at::Tensor& x, const at::Tensor& weight, bool b_mn, const at::Tensor& peer_stage_ptrs,
             const at::Tensor& peer_count_ptrs, at::Tensor& out, const at::Tensor& epoch, int64_t rank, int64_t tp) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kBFloat16);
  TORCH_CHECK(weight.scalar_type() == at::kBFloat16 && weight.dim() == 2 && weight.stride(1) == 1);
  TORCH_CHECK(tp >= 2 && tp <= COMM_MAX_RANKS && peer_stage_ptrs.numel() == tp && peer_count_ptrs.numel() == tp);
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), K = x.size(1);
  const int Kb = b_mn ? weight.size(0) : weight.size(1);
  const int N = b_mn ? weight.size(1) : weight.size(0);
  TORCH_CHECK(K == Kb && T % (tp * GEMM_BM) == 0 && N % 64 == 0, "gemm_rs: N must be a multiple of 64");
  TORCH_CHECK(out.is_contiguous() && out.size(0) == T / tp && out.size(1) == N && out.scalar_type() == at::kBFloat16);
  const int BN = pick_bn(T, N, false, sms());
  GemmParams p;
  p.M = T; p.N = N; p.K = K;
  p.D = nullptr; p.ldd = N; p.D2 = nullptr; p.ldd2 = 0;
  p.m_blocks = T / GEMM_BM; p.n_blocks = (N + BN - 1) / BN; p.k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.group_m = 4;
  p.block_expert = nullptr; p.n_per_expert = 0; p.expert_rows = nullptr; p.tiles_per_expert = 0; p.d_expert_stride = 0;
  p.status = status_word();
  CommParams c{};
  c.mode = MODE_RS; c.rank = rank; c.tp = tp; c.rows_per_rank = T / tp; c.epoch_ptr = epoch.data_ptr<int>(); c.n_copy_ctas = 0;
  for (int q = 0; q < tp; ++q) {
    c.peer_stage[q] = reinterpret_cast<__nv_bfloat16*>(peer_stage_ptrs.data_ptr<int64_t>()[q]);
    c.peer_count[q] = reinterpret_cast<int*>(peer_count_ptrs.data_ptr<int64_t>()[q]);
  }
  c.stage = c.peer_stage[rank];
  c.count = c.peer_count[rank];
  c.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  c.tiles_per_source = (c.rows_per_rank / GEMM_BM) * p.n_blocks;
  // transport of the partial tiles: the producers push them into the owner's staging (default) or the owner pulls them
  // from the producers' staging (PFB_RS_PULL=1); every rank of a group must use the same setting
  static const bool pull = [] { const char* e = std::getenv("PFB_RS_PULL"); return e && e[0] == '1'; }();
  c.pull = pull ? 1 : 0;
  CUtensorMap tmA = make_tma_2d(x.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, K, x.stride(0), GEMM_BM, 64);
  CUtensorMap tmB = b_mn ? make_tma_2d(weight.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, weight.stride(0), GEMM_BK, 64)
                         : make_tma_2d(weight.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, weight.stride(0), BN, 64);
  const int tiles = p.m_blocks * p.n_blocks;
  const int grid = std::min(tiles, sms());
  StageMaps sm{};
  for (int q = 0; q < COMM_MAX_RANKS; ++q)
    sm.m[q] = make_tma_2d(c.peer_stage[q < tp ? q : 0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, N, N, 32, 64);
  dispatch_comm<MODE_RS>(BN, b_mn, EPI_STORE_BF16, tmA, tmB, sm, p, c, grid, at::cuda::getCurrentCUDAStream());
  count_launch();
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("ag_gemm(Tensor G, Tensor peer_G_ptrs, Tensor weight, Tensor(a!) out, Tensor? out2, int epi, bool b_mn, int ready_ptr, "
        "Tensor peer_ready_ptrs, Tensor(b!) blk_flags, Tensor epoch, int rank, int tp, int n_copy) -> ()", &pfb::ag_gemm);
  m.def("gemm_rs(Tensor x, Tensor weight, bool b_mn, Tensor peer_stage_ptrs, Tensor peer_count_ptrs, Tensor(a!) out, Tensor epoch, "
        "int rank, int tp) -> ()", &pfb::gemm_rs);
}
