// Host launcher and torch binding for the tcgen05 flash attention backward (see attention_bwd_sm100.cuh).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "attention_bwd_sm100.cuh"
#include "status.h"
#include "tma_host.h"

#include <cstdlib>
#include <string>

namespace pfb {

static CUtensorMap map3(const at::Tensor& t, int box_rows) {
  TORCH_CHECK(t.dim() == 3 && t.stride(2) == 1 && t.scalar_type() == at::kBFloat16 && (t.size(2) == ATT_D || t.size(2) == 192));
  return make_tma_3d(t.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t.size(0), t.size(1), t.size(2), t.stride(0),
                     t.stride(1), box_rows, 1, 64);
}

// dout, q, out: [B,S,Hq,128]; k, v: [B,S,Hkv,128] (q/k/v/dq/dk/dv may be strided views of packed buffers);
// lse: [B,Hq,S]. Writes dq, dk, dv.
void attn_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& out,
              const at::Tensor& lse, at::Tensor& dq, at::Tensor& dk, at::Tensor& dv, int64_t B, int64_t S, double scale,
              bool causal, const c10::optional<at::Tensor>& kend, const c10::optional<at::Tensor>& tile_min,
              const c10::optional<at::Tensor>& tile_max, bool deterministic, int64_t heads_per_cta_override) {
  const int DQK = q.size(-1);
  TORCH_CHECK(q.is_cuda() && (DQK == ATT_D || DQK == 192) && k.size(-1) == DQK && v.size(-1) == ATT_D,
              "attn_bwd: queries / keys 128 or 192 wide, values 128 wide");
  const c10::cuda::CUDAGuard guard(q.device());
  const int Hq = q.size(-2), Hkv = k.size(-2);
  TORCH_CHECK(DQK == ATT_D || Hq == Hkv, "attn_bwd: 192-wide heads need as many key heads as query heads");
  const long long T = B * S;
  at::Tensor q3 = q.view({T, Hq, DQK}), k3 = k.view({T, Hkv, DQK}), v3 = v.view({T, Hkv, ATT_D});
  at::Tensor do3 = dout.contiguous().view({T, Hq, ATT_D});
  at::Tensor o3 = out.contiguous().view({T, Hq, ATT_D});
  at::Tensor dq3 = dq.view({T, Hq, DQK}), dk3 = dk.view({T, Hkv, DQK}), dv3 = dv.view({T, Hkv, ATT_D});
  TORCH_CHECK(dq3.stride(2) == 1 && dq3.stride(1) == DQK && dk3.stride(1) == DQK && dv3.stride(1) == ATT_D);
  TORCH_CHECK(lse.is_contiguous() && lse.scalar_type() == at::kFloat);
  if (T == 0) return;
  bool group_mode = false;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  at::Tensor delta = at::empty({B, Hq, S}, lse.options());
  at::Tensor dq_acc = at::zeros({T, Hq, DQK}, lse.options());
  {
    const long long warps = T * Hq;
    attn_bwd_delta_kernel<<<static_cast<int>((warps * 32 + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(do3.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(o3.data_ptr()),
        delta.data_ptr<float>(), B, S, Hq);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  AttnBwdParams p;
  p.lse = lse.data_ptr<float>(); p.delta = delta.data_ptr<float>(); p.dq_acc = dq_acc.data_ptr<float>();
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk3.data_ptr()); p.dv = reinterpret_cast<__nv_bfloat16*>(dv3.data_ptr());
  p.dk_row_stride = dk3.stride(0); p.dv_row_stride = dv3.stride(0);
  at::Tensor dk_part, dv_part;
  p.dk_part = nullptr; p.dv_part = nullptr;
  static const bool use_v1 = [] { const char* e = std::getenv("PFB_ATTN_BWD"); return e != nullptr && std::string(e) == "v1"; }();
  // one CTA per (key tile, KV head), walking the group's query heads, when that still fills the GPU about twice over;
  // otherwise one CTA per query head with fp32 dK / dV partials that a second kernel sums
  const int G = Hq / Hkv;
  const long long group_ctas = ((S + ATTB_BKV - 1) / ATTB_BKV) * static_cast<long long>(Hkv) * B;
  int heads_per_cta = (G > 1 && group_ctas >= 2LL * at::cuda::getCurrentDeviceProperties()->multiProcessorCount) ? G : 1;
  if (heads_per_cta_override > 0) heads_per_cta = heads_per_cta_override == 1 ? 1 : G;
  if (use_v1 || DQK != ATT_D) heads_per_cta = 1;
  group_mode = heads_per_cta != 1;
  if (Hq != Hkv && !group_mode) {
    dk_part = at::empty({T, Hq, ATT_D}, lse.options());
    dv_part = at::empty({T, Hq, ATT_D}, lse.options());
    p.dk_part = dk_part.data_ptr<float>(); p.dv_part = dv_part.data_ptr<float>();
  }
  p.kend = nullptr; p.tile_min_end = nullptr; p.tile_max_end = nullptr;
  const int kv_tiles = (S + ATTB_BKV - 1) / ATTB_BKV;
  if (kend.has_value()) {
    TORCH_CHECK(tile_min.has_value() && tile_max.has_value() && kend->scalar_type() == at::kInt && kend->is_contiguous());
    TORCH_CHECK(tile_min->numel() == B * kv_tiles && tile_max->numel() == B * kv_tiles);
    p.kend = kend->data_ptr<int>(); p.tile_min_end = tile_min->data_ptr<int>(); p.tile_max_end = tile_max->data_ptr<int>();
  }
  p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = static_cast<float>(scale); p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.causal = causal ? 1 : 0;
  p.status = status_word();
  CUtensorMap tmQ = map3(q3, ATTB_BQ), tmK = map3(k3, ATTB_BKV), tmV = map3(v3, ATTB_BKV), tmdO = map3(do3, ATTB_BQ);
  if (DQK == 192) {
    // multi-head latent attention: the one-tile-at-a-time kernel (dK alone takes 192 TMEM columns)
    static bool cfg = false;
    if (!cfg) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<192>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnBwdSmemT<192>::TOTAL));
      cfg = true;
    }
    dim3 grid(kv_tiles, Hq, B);
    attn_bwd_kernel<192><<<grid, ATTB_THREADS, AttnBwdSmemT<192>::TOTAL, stream>>>(tmQ, tmK, tmV, tmdO, p);
  } else if (use_v1) {
    static bool cfg = false;
    if (!cfg) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnBwdSmem::TOTAL));
      cfg = true;
    }
    dim3 grid(kv_tiles, Hq, B);
    attn_bwd_kernel<128><<<grid, ATTB_THREADS, AttnBwdSmem::TOTAL, stream>>>(tmQ, tmK, tmV, tmdO, p);
  } else {
    AttnBwd2Params pp;
    pp.base = p;
    pp.deterministic = deterministic ? 1 : 0;
    pp.dq_turn = nullptr;
    at::Tensor turns;
    if (deterministic) {
      turns = at::zeros({B, Hq, (S + ATTB_BQ - 1) / ATTB_BQ}, lse.options().dtype(at::kInt));
      pp.dq_turn = turns.data_ptr<int>();
    }
    pp.heads_per_cta = heads_per_cta;
    CUtensorMap tmdQ = make_tma_3d(dq_acc.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, T, Hq, ATT_D,
                                   static_cast<uint64_t>(Hq) * ATT_D, ATT_D, 32, 1, ATT_D, CU_TENSOR_MAP_SWIZZLE_NONE);
    static bool cfg = false;
    if (!cfg) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnBwd2Smem::TOTAL));
      cfg = true;
    }
    dim3 grid(kv_tiles, pp.heads_per_cta == 1 ? Hq : Hkv, B);
    attn_bwd2_kernel<<<grid, AB2_THREADS, AttnBwd2Smem::TOTAL, stream>>>(tmQ, tmK, tmV, tmdO, tmdQ, pp);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  {
    const long long work = T * (Hq * ATT_D / 4);
    const int blocks = static_cast<int>(std::min<long long>((work + 255) / 256, static_cast<long long>(at::cuda::getCurrentDeviceProperties()->multiProcessorCount) * 16));
    attn_bwd_dq_convert_kernel<<<blocks, 256, 0, stream>>>(dq_acc.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(dq3.data_ptr()),
                                                          T, Hq * DQK, dq3.stride(0));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  int launches = 3;
  if (Hq != Hkv && !group_mode) {
    const long long work = T * (Hkv * ATT_D / 4);
    const int blocks = static_cast<int>(std::min<long long>((work + 255) / 256, static_cast<long long>(at::cuda::getCurrentDeviceProperties()->multiProcessorCount) * 16));
    attn_bwd_dkv_reduce_kernel<<<blocks, 256, 0, stream>>>(dk_part.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(dk3.data_ptr()),
                                                          T, Hq, Hkv, dk3.stride(0));
    attn_bwd_dkv_reduce_kernel<<<blocks, 256, 0, stream>>>(dv_part.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(dv3.data_ptr()),
                                                          T, Hq, Hkv, dv3.stride(0));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    launches += 2;
  }
  count_launch(launches);
}

}  // namespace pfb

TORCH_LIBRARY_FRAGMENT(pfb200, m) {
  m.def("attn_bwd(Tensor dout, Tensor q, Tensor k, Tensor v, Tensor out, Tensor lse, Tensor(a!) dq, Tensor(b!) dk, "
        "Tensor(c!) dv, int B, int S, float scale, bool causal, Tensor? kend, Tensor? tile_min, Tensor? tile_max, "
        "bool deterministic=False, int heads_per_cta=0) -> ()",
        &pfb::attn_bwd);
}
