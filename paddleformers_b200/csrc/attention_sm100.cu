// Host launcher and torch binding for the tcgen05 flash attention kernels (see attention_sm100.cuh).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention_sm100.cuh"
#include "status.h"
#include "tma_host.h"

#include <cstdlib>
#include <string>

namespace pfb {

static CUtensorMap qkv_map(const at::Tensor& t, int box_rows) {
  // t: [T, H, D] view with D contiguous; strides may come from a fused qkv buffer.
  TORCH_CHECK(t.dim() == 3 && t.stride(2) == 1 && t.scalar_type() == at::kBFloat16);
  return make_tma_3d(t.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t.size(0), t.size(1), t.size(2), t.stride(0),
                     t.stride(1), box_rows, 1, 64);
}

// q: [B*S, Hq, 128], k/v: [B*S, Hkv, 128] (strided views allowed), out: [B*S, Hq, 128] contiguous rows.
// kend: optional int32 [B, S]; tile_min/max: int32 [B, ceil(S/128)] (min / max of kend per key tile).
// Returns lse [B, Hq, S] (natural log).
at::Tensor attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& out, int64_t B,
                    int64_t S, double scale, bool causal, const c10::optional<at::Tensor>& kend,
                    const c10::optional<at::Tensor>& tile_min, const c10::optional<at::Tensor>& tile_max,
                    bool p_in_tmem) {
  const int DQK = q.size(2);
  TORCH_CHECK(q.is_cuda() && (DQK == ATT_D || DQK == 192) && k.size(2) == DQK && v.size(2) == ATT_D,
              "attn_fwd: queries / keys 128 or 192 wide, values 128 wide");
  TORCH_CHECK(q.size(0) == B * S && k.size(0) == B * S && v.size(0) == B * S);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 3 && out.stride(2) == 1 && out.stride(1) == ATT_D);
  const c10::cuda::CUDAGuard guard(q.device());
  const int Hq = q.size(1), Hkv = k.size(1);
  TORCH_CHECK(Hq % Hkv == 0 && v.size(1) == Hkv);
  at::Tensor lse = at::empty({B, Hq, S}, q.options().dtype(at::kFloat));
  if (B * S == 0) return lse;
  AttnFwdParams p;
  p.O = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.lse = lse.data_ptr<float>();
  p.kend = nullptr; p.tile_min_end = nullptr; p.tile_max_end = nullptr;
  const int kv_tiles = (S + ATT_BKV - 1) / ATT_BKV;
  if (kend.has_value()) {
    TORCH_CHECK(tile_min.has_value() && tile_max.has_value());
    TORCH_CHECK(kend->scalar_type() == at::kInt && kend->is_contiguous() && kend->numel() == B * S);
    TORCH_CHECK(tile_min->scalar_type() == at::kInt && tile_min->is_contiguous() && tile_min->numel() == B * kv_tiles);
    TORCH_CHECK(tile_max->scalar_type() == at::kInt && tile_max->is_contiguous() && tile_max->numel() == B * kv_tiles);
    p.kend = kend->data_ptr<int>(); p.tile_min_end = tile_min->data_ptr<int>(); p.tile_max_end = tile_max->data_ptr<int>();
  }
  p.o_row_stride = out.stride(0);
  p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.causal = causal ? 1 : 0;
  p.status = status_word();
  CUtensorMap tmQ = qkv_map(q, ATT_BQ), tmK = qkv_map(k, ATT_BKV), tmV = qkv_map(v, ATT_BKV);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  static const bool use_v1 = [] { const char* e = std::getenv("PFB_ATTN_FWD"); return e != nullptr && std::string(e) == "v1"; }();
  if (DQK == 192) {
    // multi-head latent attention (192-wide queries / keys, 128-wide values): one query tile per CTA
    auto kern = attn_fwd_kernel<true, 192>;
    constexpr int smem = AttnFwdSmem<true, 192>::TOTAL;
    static bool cfg = false;
    if (!cfg) { C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); cfg = true; }
    dim3 grid1((S + ATT_BQ - 1) / ATT_BQ, Hq, B);
    kern<<<grid1, ATT_THREADS, smem, stream>>>(tmQ, tmK, tmV, p);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    return lse;
  }
  if (!use_v1) {
    // two query tiles per CTA, softmax of one tile under the products of the other
    constexpr int smem = AttnFwd2Smem::TOTAL;
    static bool cfg = false;
    if (!cfg) { C10_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); cfg = true; }
    dim3 grid2((S + 2 * ATT_BQ - 1) / (2 * ATT_BQ), Hq, B);
    attn_fwd2_kernel<<<grid2, AF2_THREADS, smem, stream>>>(tmQ, tmK, tmV, p);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    return lse;
  }
  dim3 grid((S + ATT_BQ - 1) / ATT_BQ, Hq, B);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return lse;
}

}  // namespace pfb
