// Torch bindings for the memory-bound kernels (norm / activation / rope / loss / optimizer / embedding).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "loss_optim.cuh"
#include "norm_act.cuh"
#include "status.h"

namespace pfb {

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }
static inline const __nv_bfloat16* bf(const at::Tensor& t) { return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr()); }
static inline __nv_bfloat16* bfm(at::Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }
static int num_sms() {
  static int n = 0;
  if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}
static int ew_grid(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  long long cap = static_cast<long long>(num_sms()) * 16;
  return static_cast<int>(std::max(1LL, std::min(b, cap)));
}

// y, rstd = rms_norm(x [+ residual]); when residual is given also returns the sum (new residual stream).
std::tuple<at::Tensor, at::Tensor, at::Tensor> rms_norm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& residual,
                                                             const at::Tensor& w, double eps) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1);
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), H = x.size(1);
  TORCH_CHECK(H % 8 == 0 && x.stride(0) % 8 == 0 && w.numel() == H && w.scalar_type() == at::kBFloat16);
  at::Tensor y = at::empty({T, H}, x.options());
  at::Tensor rstd = at::empty({T}, x.options().dtype(at::kFloat));
  at::Tensor sum;
  if (residual.has_value()) {
    TORCH_CHECK(residual->is_contiguous() && residual->sizes() == x.sizes());
    sum = at::empty({T, H}, x.options());
  }
  if (T > 0) {
    const int threads = H >= 2048 ? 256 : 128;
    rms_norm_fwd_kernel<<<T, threads, 0, cur_stream()>>>(bf(x), residual.has_value() ? bf(*residual) : nullptr, bf(w),
                                                        bfm(y), residual.has_value() ? bfm(sum) : nullptr,
                                                        rstd.data_ptr<float>(), H, x.stride(0), H, static_cast<float>(eps));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
  }
  return {y, rstd, sum};
}

// dx (+= dres), dw: dw is accumulated into `dw_out` (fp32 [H]) when accumulate is true, else overwritten.
// `scratch` is a caller-provided fp32 buffer of at least rms_norm_bwd_scratch_rows() * H elements.
int64_t rms_norm_bwd_scratch_rows() { return static_cast<int64_t>(num_sms()) * 4; }

at::Tensor rms_norm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd,
                        const c10::optional<at::Tensor>& dres, at::Tensor& dw_out, bool accumulate,
                        at::Tensor& scratch) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.dim() == 2 && dy.stride(1) == 1);
  TORCH_CHECK(x.is_contiguous() && dw_out.scalar_type() == at::kFloat && scratch.scalar_type() == at::kFloat);
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), H = x.size(1);
  TORCH_CHECK(H % 8 == 0 && H <= 16384, "rms_norm_bwd: H % 8 == 0 and H <= 16384");
  at::Tensor dx = at::empty({T, H}, x.options());
  const int P = static_cast<int>(std::min<int64_t>(rms_norm_bwd_scratch_rows(), std::max(T, 1)));
  TORCH_CHECK(scratch.numel() >= static_cast<int64_t>(P) * H, "rms_norm_bwd: scratch too small");
  if (T == 0) return dx;
  const __nv_bfloat16* dr = dres.has_value() ? bf(*dres) : nullptr;
  const int threads = 256;
  const int per = (H / 8 + threads - 1) / threads;
  auto launch = [&](auto tag) {
    constexpr int PT = decltype(tag)::value;
    rms_norm_bwd_kernel<PT><<<P, threads, 0, cur_stream()>>>(bf(dy), bf(x), bf(w), rstd.data_ptr<float>(), dr, bfm(dx),
                                                           scratch.data_ptr<float>(), T, H, dy.stride(0));
  };
  if (per <= 1) launch(std::integral_constant<int, 1>{});
  else if (per <= 2) launch(std::integral_constant<int, 2>{});
  else if (per <= 4) launch(std::integral_constant<int, 4>{});
  else launch(std::integral_constant<int, 8>{});
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  rms_norm_dw_reduce_kernel<<<(H + 31) / 32, 256, 0, cur_stream()>>>(scratch.data_ptr<float>(), dw_out.data_ptr<float>(),
                                                                      P, H, accumulate ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
  return dx;
}

at::Tensor swiglu_fwd(const at::Tensor& gu) {
  TORCH_CHECK(gu.is_cuda() && gu.scalar_type() == at::kBFloat16 && gu.dim() == 2 && gu.stride(1) == 1);
  const c10::cuda::CUDAGuard guard(gu.device());
  const long long T = gu.size(0);
  const int I = gu.size(1) / 2;
  TORCH_CHECK(I % 8 == 0 && gu.stride(0) % 8 == 0);
  at::Tensor act = at::empty({T, I}, gu.options());
  if (T == 0) return act;
  swiglu_fwd_kernel<<<ew_grid(T * (I / 8), 256), 256, 0, cur_stream()>>>(bf(gu), bfm(act), T, I, gu.stride(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return act;
}

std::tuple<at::Tensor, at::Tensor> swiglu_bwd(const at::Tensor& dact, const at::Tensor& gu, bool want_act) {
  TORCH_CHECK(gu.is_cuda() && gu.scalar_type() == at::kBFloat16 && gu.dim() == 2 && gu.stride(1) == 1);
  TORCH_CHECK(dact.is_contiguous() && dact.scalar_type() == at::kBFloat16);
  const c10::cuda::CUDAGuard guard(gu.device());
  const long long T = gu.size(0);
  const int I = gu.size(1) / 2;
  at::Tensor dgu = at::empty({T, 2 * I}, gu.options());
  at::Tensor act;
  if (want_act) act = at::empty({T, I}, gu.options());
  if (T == 0) return {dgu, act};
  swiglu_bwd_kernel<<<ew_grid(T * (I / 8), 256), 256, 0, cur_stream()>>>(bf(dact), bf(gu), bfm(dgu),
                                                                         want_act ? bfm(act) : nullptr, T, I, gu.stride(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dgu, act};
}

// In-place rotary embedding on x viewed as [T, n_heads, D] with row stride x.stride(0).
void rope_inplace(at::Tensor& x, const c10::optional<at::Tensor>& pos, const at::Tensor& cos, const at::Tensor& sin,
                  int64_t n_heads, int64_t D, int64_t rot, bool backward) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1);
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.is_contiguous() && sin.is_contiguous());
  TORCH_CHECK(cos.size(-1) == rot / 2 && x.size(1) >= n_heads * D && rot <= D && rot % 2 == 0);
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0);
  if (T == 0) return;
  const int* pp = nullptr;
  if (pos.has_value()) { TORCH_CHECK(pos->scalar_type() == at::kInt && pos->numel() == T); pp = pos->data_ptr<int>(); }
  else TORCH_CHECK(cos.size(0) >= T, "rope: cos/sin table shorter than the sequence");
  const long long work = static_cast<long long>(T) * n_heads * (rot / 2);
  const bool vec = rot % 16 == 0 && D % 8 == 0 && x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0;
  if (vec)
    rope_vec8_kernel<<<ew_grid(work / 8, 256), 256, 0, cur_stream()>>>(bfm(x), pp, cos.data_ptr<float>(), sin.data_ptr<float>(), T,
                                                                      static_cast<int>(n_heads), static_cast<int>(D),
                                                                      static_cast<int>(rot), x.stride(0), backward ? -1.f : 1.f);
  else
    rope_kernel<<<ew_grid(work, 256), 256, 0, cur_stream()>>>(bfm(x), pp, cos.data_ptr<float>(), sin.data_ptr<float>(), T,
                                                             static_cast<int>(n_heads), static_cast<int>(D),
                                                             static_cast<int>(rot), x.stride(0), backward ? -1.f : 1.f);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

// out = rope(rmsnorm_D(x) * nw): x, out viewed as [T, n_heads, D]; returns rstd [T, n_heads].
at::Tensor qk_norm_rope_fwd(const at::Tensor& x, at::Tensor& out, const at::Tensor& nw,
                            const c10::optional<at::Tensor>& pos, const at::Tensor& cos, const at::Tensor& sin,
                            int64_t n_heads, int64_t D, int64_t rot, double eps) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1);
  TORCH_CHECK(D <= 256 && rot <= D && rot % 2 == 0 && nw.numel() == D);
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0);
  at::Tensor rstd = at::empty({T, n_heads}, x.options().dtype(at::kFloat));
  if (T == 0) return rstd;
  const int* pp = pos.has_value() ? pos->data_ptr<int>() : nullptr;
  const long long warps = static_cast<long long>(T) * n_heads;
  const int threads = 256;
  auto aligned8 = [](const at::Tensor& t) { return (reinterpret_cast<uintptr_t>(t.data_ptr()) & 7) == 0 && t.stride(0) % 4 == 0; };
  if (D == 128 && rot == 128 && aligned8(x) && aligned8(out) && (reinterpret_cast<uintptr_t>(nw.data_ptr()) & 7) == 0) {
    // 128-wide heads with full rotary: 8-byte accesses, warps stride over the (token, head) pairs
    const int blocks = static_cast<int>(std::min<long long>((warps * 32 + threads - 1) / threads, static_cast<long long>(num_sms()) * 16));
    qk_norm_rope_fwd128_kernel<<<blocks, threads, 0, cur_stream()>>>(
        bf(x), bfm(out), bf(nw), rstd.data_ptr<float>(), pp, cos.data_ptr<float>(), sin.data_ptr<float>(), T,
        static_cast<int>(n_heads), x.stride(0), out.stride(0), static_cast<float>(eps));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    return rstd;
  }
  qk_norm_rope_fwd_kernel<<<static_cast<int>((warps * 32 + threads - 1) / threads), threads, 0, cur_stream()>>>(
      bf(x), bfm(out), bf(nw), rstd.data_ptr<float>(), pp, cos.data_ptr<float>(), sin.data_ptr<float>(), T,
      static_cast<int>(n_heads), static_cast<int>(D), static_cast<int>(rot), x.stride(0), out.stride(0),
      static_cast<float>(eps));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return rstd;
}

void qk_norm_rope_bwd(const at::Tensor& dout, const at::Tensor& x, const at::Tensor& nw, const at::Tensor& rstd,
                      at::Tensor& dx, at::Tensor& dnw, const c10::optional<at::Tensor>& pos, const at::Tensor& cos,
                      const at::Tensor& sin, int64_t n_heads, int64_t D, int64_t rot) {
  TORCH_CHECK(dout.is_cuda() && dout.stride(1) == 1 && x.stride(1) == 1 && dx.stride(1) == 1);
  TORCH_CHECK(dnw.scalar_type() == at::kFloat && dnw.numel() == D && D <= 256);
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0);
  if (T == 0) return;
  const int* pp = pos.has_value() ? pos->data_ptr<int>() : nullptr;
  auto aligned8 = [](const at::Tensor& t) { return (reinterpret_cast<uintptr_t>(t.data_ptr()) & 7) == 0 && t.stride(0) % 4 == 0; };
  if (D == 128 && rot == 128 && aligned8(dout) && aligned8(x) && aligned8(dx) && (reinterpret_cast<uintptr_t>(nw.data_ptr()) & 7) == 0) {
    qk_norm_rope_bwd128_kernel<<<num_sms() * 8, 256, 0, cur_stream()>>>(
        bf(dout), bf(x), bf(nw), rstd.data_ptr<float>(), bfm(dx), dnw.data_ptr<float>(), pp, cos.data_ptr<float>(),
        sin.data_ptr<float>(), T, static_cast<int>(n_heads), dout.stride(0), x.stride(0), dx.stride(0));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    return;
  }
  qk_norm_rope_bwd_kernel<<<num_sms() * 4, 256, 0, cur_stream()>>>(
      bf(dout), bf(x), bf(nw), rstd.data_ptr<float>(), bfm(dx), dnw.data_ptr<float>(), pp, cos.data_ptr<float>(),
      sin.data_ptr<float>(), T, static_cast<int>(n_heads), static_cast<int>(D), static_cast<int>(rot), dout.stride(0),
      x.stride(0), dx.stride(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

// mode 0: loss + in-place grad (single vocabulary shard). mode 1: write (max, sumexp, label logit) partials.
// mode 2: in-place grad from reduced (max, sum) statistics.
void cross_entropy(at::Tensor& logits, const at::Tensor& labels, at::Tensor& loss, at::Tensor& stat_max,
                   at::Tensor& stat_sum, at::Tensor& stat_label, const at::Tensor& grad_scale, int64_t vocab_start,
                   int64_t ignore_index, int64_t mode, bool write_grad) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0));
  TORCH_CHECK(grad_scale.scalar_type() == at::kFloat);
  const c10::cuda::CUDAGuard guard(logits.device());
  const int rows = logits.size(0), V = logits.size(1);
  TORCH_CHECK(V % 8 == 0 && logits.stride(0) % 8 == 0, "cross_entropy: vocab (shard) size must be a multiple of 8");
  if (rows == 0) return;
  cross_entropy_kernel<<<rows, 512, 0, cur_stream()>>>(bfm(logits), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                                                      loss.data_ptr<float>(), stat_max.data_ptr<float>(),
                                                      stat_sum.data_ptr<float>(), stat_label.data_ptr<float>(),
                                                      grad_scale.data_ptr<float>(), V, logits.stride(0),
                                                      static_cast<int>(vocab_start), ignore_index,
                                                      static_cast<int>(mode), write_grad ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

at::Tensor embedding_fwd(const at::Tensor& ids, const at::Tensor& W, int64_t vocab_start) {
  TORCH_CHECK(W.is_cuda() && W.scalar_type() == at::kBFloat16 && W.is_contiguous() && ids.scalar_type() == at::kLong);
  const c10::cuda::CUDAGuard guard(W.device());
  at::Tensor idc = ids.contiguous();
  const int T = idc.numel(), H = W.size(1);
  TORCH_CHECK(H % 8 == 0);
  at::Tensor out = at::empty({T, H}, W.options());
  if (T == 0) return out;
  embedding_fwd_kernel<<<ew_grid(static_cast<long long>(T) * (H / 8), 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<const long long*>(idc.data_ptr<int64_t>()), bf(W), bfm(out), T, H, static_cast<int>(vocab_start),
      static_cast<int>(W.size(0)));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

void embedding_bwd(const at::Tensor& ids, const at::Tensor& dout, at::Tensor& grad, int64_t vocab_start) {
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == at::kFloat && grad.is_contiguous());
  TORCH_CHECK(dout.scalar_type() == at::kBFloat16 && dout.is_contiguous());
  const c10::cuda::CUDAGuard guard(grad.device());
  at::Tensor idc = ids.contiguous();
  const int T = idc.numel(), H = grad.size(1);
  if (T == 0) return;
  embedding_bwd_kernel<<<ew_grid(static_cast<long long>(T) * (H / 2), 256), 256, 0, cur_stream()>>>(
      reinterpret_cast<const long long*>(idc.data_ptr<int64_t>()), bf(dout), grad.data_ptr<float>(), T, H,
      static_cast<int>(vocab_start), static_cast<int>(grad.size(0)));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void adamw_step(at::Tensor& p, at::Tensor& m, at::Tensor& v, const at::Tensor& g, const c10::optional<at::Tensor>& p16,
                const at::Tensor& scalars, double beta1, double beta2, double eps, double wd) {
  TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat &&
              g.scalar_type() == at::kFloat);
  TORCH_CHECK(p.is_contiguous() && m.is_contiguous() && v.is_contiguous() && g.is_contiguous());
  TORCH_CHECK(scalars.scalar_type() == at::kFloat && scalars.numel() >= 5);
  const c10::cuda::CUDAGuard guard(p.device());
  const long long n = p.numel();
  TORCH_CHECK(m.numel() == n && v.numel() == n && g.numel() == n);
  __nv_bfloat16* p16p = nullptr;
  if (p16.has_value()) {
    TORCH_CHECK(p16->scalar_type() == at::kBFloat16 && p16->numel() == n && p16->is_contiguous());
    p16p = reinterpret_cast<__nv_bfloat16*>(p16->data_ptr());
  }
  if (n == 0) return;
  adamw_kernel<<<ew_grid(n / 4 + 1, 256), 256, 0, cur_stream()>>>(p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                                                                 g.data_ptr<float>(), p16p, n, scalars.data_ptr<float>(),
                                                                 static_cast<float>(beta1), static_cast<float>(beta2),
                                                                 static_cast<float>(eps), static_cast<float>(wd));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

// out[0] += sum(x^2); `scratch` >= sq_norm_scratch_elems() floats.
int64_t sq_norm_scratch_elems() { return static_cast<int64_t>(num_sms()) * 8; }
void sq_norm_accum(const at::Tensor& x, at::Tensor& out, at::Tensor& scratch) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous() && out.scalar_type() == at::kFloat);
  const c10::cuda::CUDAGuard guard(x.device());
  const long long n = x.numel();
  if (n == 0) return;
  const int P = static_cast<int>(std::min<long long>(sq_norm_scratch_elems(), (n / 4 + 255) / 256 + 1));
  TORCH_CHECK(scratch.numel() >= P && scratch.scalar_type() == at::kFloat);
  sq_norm_partial_kernel<<<P, 256, 0, cur_stream()>>>(x.data_ptr<float>(), n, scratch.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  sq_norm_finish_kernel<<<1, 256, 0, cur_stream()>>>(scratch.data_ptr<float>(), P, out.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
}

void cast_scale(const at::Tensor& src, at::Tensor& dst, double scale, bool accumulate) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel());
  const c10::cuda::CUDAGuard guard(src.device());
  const long long n = src.numel();
  if (n == 0) return;
  if (src.scalar_type() == at::kFloat && dst.scalar_type() == at::kBFloat16) {
    cast_f32_to_bf16_kernel<<<ew_grid(n, 256), 256, 0, cur_stream()>>>(src.data_ptr<float>(), bfm(dst), n, static_cast<float>(scale));
  } else if (src.scalar_type() == at::kBFloat16 && dst.scalar_type() == at::kFloat) {
    accum_bf16_to_f32_kernel<<<ew_grid(n, 256), 256, 0, cur_stream()>>>(bf(src), dst.data_ptr<float>(), n, static_cast<float>(scale), accumulate ? 1 : 0);
  } else {
    TORCH_CHECK(false, "cast_scale: fp32->bf16 or bf16->fp32 only");
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace pfb
