// Host launcher and torch binding for the tcgen05 bf16 GEMM family (see gemm_sm100.cuh).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "gemm2_sm100.cuh"
#include "gemm_sm100.cuh"

#include <cstdlib>
#include <string>
#include "status.h"
#include "tma_host.h"

namespace pfb {

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI, bool GROUPED, bool KGROUPED = false>
static void launch_one(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid,
                       cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, EPI, GROUPED, KGROUPED>;
  constexpr int smem = GemmSmem<BN, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, smem, stream>>>(tmA, tmB, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <int BN, int STAGES>
static void dispatch(bool a_mn, bool b_mn, int epi, bool grouped, const CUtensorMap& tmA, const CUtensorMap& tmB,
                     const GemmParams& p, int grid, cudaStream_t s) {
#define PFB_CASE(AMN, BMN, E, G)                                                      \
  if (a_mn == AMN && b_mn == BMN && epi == E && grouped == G) {                       \
    launch_one<BN, STAGES, AMN, BMN, E, G>(tmA, tmB, p, grid, s);                     \
    return;                                                                           \
  }
  PFB_CASE(false, false, EPI_STORE_BF16, false)
  PFB_CASE(false, false, EPI_STORE_F32, false)
  PFB_CASE(false, false, EPI_ACCUM_BF16, false)
  PFB_CASE(false, false, EPI_SWIGLU_BF16, false)
  PFB_CASE(false, true, EPI_STORE_BF16, false)
  PFB_CASE(false, true, EPI_ACCUM_BF16, false)
  PFB_CASE(true, true, EPI_STORE_BF16, false)
  PFB_CASE(true, true, EPI_STORE_F32, false)
  PFB_CASE(true, true, EPI_ACCUM_F32, false)
  PFB_CASE(false, false, EPI_STORE_BF16, true)
  PFB_CASE(false, false, EPI_SWIGLU_BF16, true)
  PFB_CASE(false, true, EPI_STORE_BF16, true)
#undef PFB_CASE
  TORCH_CHECK(false, "pfb200::gemm: unsupported combination a_mn=", a_mn, " b_mn=", b_mn, " epi=", epi,
              " grouped=", grouped);
}

// ---- CTA-pair kernel (gemm2_sm100.cuh): launched as clusters of two CTAs
template <bool A_MN, bool B_MN, int EPI>
static void launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const GemmParams& p, int n_clusters,
                        cudaStream_t stream) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, EPI>;
  constexpr int smem = Gemm2SmemFor<EPI>::TOTAL;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * n_clusters, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  C10_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmD, p));
}

static bool dispatch_pair(bool a_mn, bool b_mn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD,
                          const GemmParams& p, int n_clusters, cudaStream_t s) {
#define PFB_PAIR(AMN, BMN, E)                                                                       \
  if (a_mn == AMN && b_mn == BMN && epi == E) { launch_pair<AMN, BMN, E>(tmA, tmB, tmD, p, n_clusters, s); return true; }
  PFB_PAIR(false, false, EPI_STORE_BF16)
  PFB_PAIR(false, false, EPI_STORE_F32)
  PFB_PAIR(false, false, EPI_ACCUM_BF16)
  PFB_PAIR(false, false, EPI_SWIGLU_BF16)
  PFB_PAIR(false, true, EPI_STORE_BF16)
  PFB_PAIR(false, true, EPI_ACCUM_BF16)
  PFB_PAIR(true, true, EPI_STORE_BF16)
  PFB_PAIR(true, true, EPI_STORE_F32)
  PFB_PAIR(true, true, EPI_ACCUM_F32)
  PFB_PAIR(true, true, EPI_REDUCE_F32)
#undef PFB_PAIR
  return false;
}

// PFB_GEMM_PAIR=0 keeps every product on the one-CTA kernel (A/B switch)
static bool pair_enabled() {
  static const bool on = [] { const char* e = std::getenv("PFB_GEMM_PAIR"); return e == nullptr || std::string(e) != "0"; }();
  return on;
}

// The fp32-accumulating weight-gradient product adds its tiles through TMA reduce operations (the sum is formed in L2)
// instead of reading the old values into the epilogue warps: +9-24 % on the model's weight-gradient shapes.
// PFB_GEMM_TMA_REDUCE=0 restores the read-add-store epilogue.
static bool tma_reduce_enabled() {
  static const bool on = [] { const char* e = std::getenv("PFB_GEMM_TMA_REDUCE"); return e == nullptr || std::string(e) != "0"; }();
  return on;
}

// When the last round of tiles would keep at most half of the CTA pairs busy, its tiles are computed as two 128-column
// halves each, which halves the length of that round (+3-7 % on products with 256 or 384 tiles). PFB_GEMM_TAIL_SPLIT=0
// switches it off.
static bool tail_split_enabled() {
  static const bool on = [] { const char* e = std::getenv("PFB_GEMM_TAIL_SPLIT"); return e == nullptr || std::string(e) != "0"; }();
  return on;
}

static int sm_count() {
  static int n = 0;
  if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

// a: [M,K] (a_mn=false) or [K,M] (a_mn=true); b: [N,K] or [K,N] (grouped: [E*N,K] or [K? no: E stacked on rows]).
// out: [M,N] (SwiGLU: [M,N/2]); dtype decides between bf16 / fp32 epilogues.
void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& out, bool a_mn, bool b_mn, int64_t epi,
          const c10::optional<at::Tensor>& out2, const c10::optional<at::Tensor>& block_expert,
          int64_t n_per_expert, int64_t force_bn) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "pfb200::gemm needs CUDA tensors");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "pfb200::gemm: bf16 inputs");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "pfb200::gemm: 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "pfb200::gemm: inner dim contiguous");
  const c10::cuda::CUDAGuard guard(a.device());
  const bool grouped = block_expert.has_value();
  const int M = a_mn ? a.size(1) : a.size(0);
  const int K = a_mn ? a.size(0) : a.size(1);
  const int Kb = b_mn ? b.size(0) : b.size(1);
  const int Nb_rows = b_mn ? b.size(1) : b.size(0);
  const int N = grouped ? static_cast<int>(n_per_expert) : Nb_rows;
  if (grouped && b_mn) {
    // stacked [E*K, N]: every expert contributes K rows of an MN-major operand
    TORCH_CHECK(Kb % K == 0 && Nb_rows == N, "grouped GEMM (MN-major B): b must be [E*K, N]");
  } else {
    TORCH_CHECK(K == Kb, "pfb200::gemm: K mismatch ", K, " vs ", Kb);
  }
  if (grouped) {
    TORCH_CHECK(!a_mn, "grouped GEMM needs a K-major A");
    TORCH_CHECK(b_mn || Nb_rows % N == 0, "grouped GEMM: stacked B rows must be a multiple of n_per_expert");
    TORCH_CHECK(block_expert->scalar_type() == at::kInt && block_expert->is_cuda());
    TORCH_CHECK(block_expert->numel() * GEMM_BM >= M, "grouped GEMM: block_expert too short");
  }
  const bool swiglu = epi == EPI_SWIGLU_BF16;
  const int N_out = swiglu ? N / 2 : N;
  TORCH_CHECK(out.size(0) == M && out.size(1) == N_out, "pfb200::gemm: out shape");
  if (epi == EPI_STORE_BF16 || epi == EPI_ACCUM_BF16 || swiglu) {
    TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.stride(0) % 8 == 0, "bf16 out, row stride % 8");
  } else {
    TORCH_CHECK(out.scalar_type() == at::kFloat && out.stride(0) % 4 == 0, "fp32 out, row stride % 4");
  }
  TORCH_CHECK((reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0, "out must be 16-byte aligned");
  if (M == 0 || N == 0) return;
  if (K == 0) {
    if (epi == EPI_STORE_BF16 || epi == EPI_STORE_F32 || swiglu) out.zero_();
    return;
  }

  // tile width: minimise waves * BN
  int BN = 256;
  if (force_bn == 128 || force_bn == 256) {
    BN = static_cast<int>(force_bn);
  } else {
    const int sms = sm_count();
    auto cost = [&](int bn) {
      int nn = swiglu ? (N_out + bn / 2 - 1) / (bn / 2) : (N + bn - 1) / bn;
      long long tiles = static_cast<long long>((M + GEMM_BM - 1) / GEMM_BM) * nn;
      return ((tiles + sms - 1) / sms) * bn;
    };
    // a 256-wide tile moves 1.33x fewer operand bytes per FLOP and measured 1.4-1.5x the rate of a 128-wide one on
    // every model shape, so the narrow tile is chosen only when it saves more than that in wave quantisation
    BN = cost(128) * 3 < cost(256) * 2 ? 128 : 256;
  }

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.D = out.data_ptr(); p.ldd = out.stride(0);
  p.D2 = nullptr; p.ldd2 = 0;
  if (out2.has_value()) {
    TORCH_CHECK(swiglu && out2->scalar_type() == at::kBFloat16 && out2->size(0) == M && out2->size(1) == N &&
                out2->stride(1) == 1 && out2->stride(0) % 8 == 0, "out2: raw [M,N] bf16 for the SwiGLU epilogue");
    p.D2 = out2->data_ptr(); p.ldd2 = out2->stride(0);
  }
  p.m_blocks = (M + GEMM_BM - 1) / GEMM_BM;
  p.n_blocks = swiglu ? (N_out + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
  p.k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.group_m = 16;
  p.block_expert = grouped ? block_expert->data_ptr<int>() : nullptr;
  p.n_per_expert = static_cast<int>(n_per_expert);
  p.expert_rows = nullptr; p.tiles_per_expert = 0; p.d_expert_stride = 0;
  p.status = status_word();

  const uint32_t b_box_rows = swiglu ? BN / 2 : BN;
  CUtensorMap tmA = a_mn ? make_tma_2d(a.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, a.stride(0), GEMM_BK, 64)
                         : make_tma_2d(a.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, a.stride(0), GEMM_BM, 64);
  CUtensorMap tmB = b_mn ? make_tma_2d(b.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Kb, Nb_rows, b.stride(0), GEMM_BK, 64)
                         : make_tma_2d(b.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Nb_rows, K, b.stride(0), b_box_rows, 64);

  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  // CTA pairs (256 x 256 tiles) whenever the problem has enough of them to fill the SM pairs about as well as the
  // one-CTA tiling would; force_bn pins the one-CTA kernel (used by the benchmarks for the A/B)
  if (!grouped && force_bn == 0 && pair_enabled() && M >= 2 * GEMM_BM && N_out >= (swiglu ? G2_HALF : G2_BN)) {
    const int pairs = sm_count() / 2;
    const int m_pairs = (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
    const int n2 = swiglu ? (N_out + G2_HALF - 1) / G2_HALF : (N + G2_BN - 1) / G2_BN;
    const long long tiles2 = static_cast<long long>(m_pairs) * n2;
    const long long waves2 = (tiles2 + pairs - 1) / pairs;
    const long long tiles1 = static_cast<long long>(p.m_blocks) * p.n_blocks;
    const long long waves1 = (tiles1 + sm_count() - 1) / sm_count();
    // time ~ waves x tile area per SM; the pair kernel runs ~1.2x faster per unit of tile area
    if (waves2 * (GEMM_BM * G2_BN) * 10 <= waves1 * (GEMM_BM * BN) * 12) {
      GemmParams p2 = p;
      p2.n_blocks = n2;
      p2.group_m = 8;
      CUtensorMap tmA2 = a_mn ? make_tma_2d(a.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, a.stride(0), GEMM_BK, 64)
                              : make_tma_2d(a.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, a.stride(0), GEMM_BM, 64);
      // B travels in 64-row boxes: two per CTA and stage for a whole tile, one for a half tile
      CUtensorMap tmB2 = b_mn ? make_tma_2d(b.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Kb, Nb_rows, b.stride(0), GEMM_BK, 64)
                              : make_tma_2d(b.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Nb_rows, K, b.stride(0), 64, 64);
      const int n_clusters = static_cast<int>(std::min<long long>(tiles2, pairs));
      const int tail = static_cast<int>(tiles2 % n_clusters);
      if (tail_split_enabled() && tiles2 > n_clusters && tail > 0 && 2 * tail <= n_clusters) p2.split_tail = tail;
      int epi2 = static_cast<int>(epi);
      CUtensorMap tmD2 = tmA2;     // only the reduce-add epilogue reads it
      if (epi2 == EPI_ACCUM_F32 && a_mn && b_mn && tma_reduce_enabled() && out.stride(0) % 4 == 0 &&
          (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0) {
        epi2 = EPI_REDUCE_F32;
        tmD2 = make_tma_2d(out.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, out.stride(0), 32, 32);
      }
      if (dispatch_pair(a_mn, b_mn, epi2, tmA2, tmB2, tmD2, p2, n_clusters, stream)) {
        count_launch();
        return;
      }
    }
  }
  const int tiles = p.m_blocks * p.n_blocks;
  const int grid = std::min(tiles, sm_count());
  if (BN == 256) dispatch<256, 4>(a_mn, b_mn, static_cast<int>(epi), grouped, tmA, tmB, p, grid, stream);
  else dispatch<128, 6>(a_mn, b_mn, static_cast<int>(epi), grouped, tmA, tmB, p, grid, stream);
  count_launch();
}


// Expert weight gradients in one launch: dW[e] (+)= dy[rows_e]^T @ x[rows_e] for every expert e.
// dy: [R, N], x: [R, K] (expert-sorted rows, segments padded to 64-row multiples with zero rows),
// expert_rows: int32 [E, 2] = (first row, row count); out: fp32 [E, N, K], accumulated in place.
void gemm_wgrad_grouped(const at::Tensor& dy, const at::Tensor& x, at::Tensor& out, const at::Tensor& expert_rows) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16);
  TORCH_CHECK(dy.dim() == 2 && x.dim() == 2 && dy.stride(1) == 1 && x.stride(1) == 1 && dy.size(0) == x.size(0));
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.dim() == 3 && out.is_contiguous());
  TORCH_CHECK(expert_rows.scalar_type() == at::kInt && expert_rows.is_contiguous() && expert_rows.is_cuda());
  const c10::cuda::CUDAGuard guard(dy.device());
  const int E = out.size(0), N = out.size(1), K = out.size(2), R = dy.size(0);
  TORCH_CHECK(dy.size(1) == N && x.size(1) == K && expert_rows.numel() == 2 * E && K % 4 == 0);
  if (E == 0 || R == 0) return;
  constexpr int BN = 256;
  GemmParams p;
  p.M = N; p.N = K; p.K = R;
  p.D = out.data_ptr(); p.ldd = K; p.D2 = nullptr; p.ldd2 = 0;
  p.m_blocks = (N + GEMM_BM - 1) / GEMM_BM;
  p.n_blocks = (K + BN - 1) / BN;
  p.k_blocks = 0;
  p.group_m = 16;
  p.block_expert = nullptr;
  p.n_per_expert = E;
  p.expert_rows = expert_rows.data_ptr<int>();
  p.tiles_per_expert = p.m_blocks * p.n_blocks;
  p.d_expert_stride = static_cast<long long>(N) * K;
  p.status = status_word();
  CUtensorMap tmA = make_tma_2d(dy.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, N, dy.stride(0), GEMM_BK, 64);
  CUtensorMap tmB = make_tma_2d(x.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, R, K, x.stride(0), GEMM_BK, 64);
  const int tiles = p.tiles_per_expert * E;
  launch_one<BN, 4, true, true, EPI_ACCUM_F32, false, true>(tmA, tmB, p, std::min(tiles, sm_count()),
                                                           at::cuda::getCurrentCUDAStream());
  count_launch();
}

}  // namespace pfb
