// Operator registration: every kernel of the extension is exposed as torch.ops.pfb200.<name>.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "status.h"

namespace pfb {

// ---- status word + launch counter -------------------------------------------------------------------------
static std::mutex g_mu;
static std::unordered_map<int, int*> g_status;
static std::atomic<int64_t> g_launches{0};

int* status_word() {
  int dev = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_status.find(dev);
  if (it != g_status.end()) return it->second;
  // 16-byte block: [0] status, [1] rows dropped by the expert-parallel dispatcher (receive buffer full), [2..3] wait budget in ns (0 = the kernels' default of one second)
  int* p = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&p, 4 * sizeof(int)));
  C10_CUDA_CHECK(cudaMemset(p, 0, 4 * sizeof(int)));
  g_status[dev] = p;
  return p;
}
// Budget of every bounded device-side wait launched from now on (stream-ordered with respect to the current stream).
void set_wait_budget(double seconds) {
  int* p = status_word();
  const long long ns = seconds > 0 ? static_cast<long long>(seconds * 1e9) : 0;
  C10_CUDA_CHECK(cudaMemcpyAsync(p + 2, &ns, sizeof(ns), cudaMemcpyHostToDevice, at::cuda::getCurrentCUDAStream()));
  C10_CUDA_CHECK(cudaStreamSynchronize(at::cuda::getCurrentCUDAStream()));
}
int read_status(bool reset) {
  int* p = status_word();
  int v = 0;
  C10_CUDA_CHECK(cudaStreamSynchronize(at::cuda::getCurrentCUDAStream()));
  C10_CUDA_CHECK(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (reset && v != 0) C10_CUDA_CHECK(cudaMemset(p, 0, sizeof(int)));
  return v;
}
// Routed (token, expert) pairs that the expert-parallel dispatcher dropped since the last reset because the destination's
// receive buffer was full (capacity-factor semantics: a dropped pair contributes nothing to the token's output).
int64_t read_drop_count(bool reset) {
  int* p = status_word();
  int v = 0;
  C10_CUDA_CHECK(cudaStreamSynchronize(at::cuda::getCurrentCUDAStream()));
  C10_CUDA_CHECK(cudaMemcpy(&v, p + 1, sizeof(int), cudaMemcpyDeviceToHost));
  if (reset && v != 0) C10_CUDA_CHECK(cudaMemset(p + 1, 0, sizeof(int)));
  return v;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int64_t launch_count(bool reset) { return reset ? g_launches.exchange(0) : g_launches.load(); }

static int64_t op_read_status(bool reset) { return read_status(reset); }
static void op_set_wait_budget(double seconds) { set_wait_budget(seconds); }
static int64_t op_launch_count(bool reset) { return launch_count(reset); }
static int64_t op_read_drop_count(bool reset) { return read_drop_count(reset); }

// ---- declarations of the ops implemented in the other translation units ---------------------------------------
void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& out, bool a_mn, bool b_mn, int64_t epi,
          const c10::optional<at::Tensor>& out2, const c10::optional<at::Tensor>& block_expert, int64_t n_per_expert,
          int64_t force_bn);
void gemm_wgrad_grouped(const at::Tensor& dy, const at::Tensor& x, at::Tensor& out, const at::Tensor& expert_rows);
at::Tensor attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& out, int64_t B, int64_t S,
                    double scale, bool causal, const c10::optional<at::Tensor>& kend,
                    const c10::optional<at::Tensor>& tile_min, const c10::optional<at::Tensor>& tile_max, bool p_in_tmem);
std::tuple<at::Tensor, at::Tensor, at::Tensor> rms_norm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& residual,
                                                             const at::Tensor& w, double eps);
int64_t rms_norm_bwd_scratch_rows();
at::Tensor rms_norm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd,
                        const c10::optional<at::Tensor>& dres, at::Tensor& dw_out, bool accumulate, at::Tensor& scratch);
at::Tensor swiglu_fwd(const at::Tensor& gu);
std::tuple<at::Tensor, at::Tensor> swiglu_bwd(const at::Tensor& dact, const at::Tensor& gu, bool want_act);
void rope_inplace(at::Tensor& x, const c10::optional<at::Tensor>& pos, const at::Tensor& cos, const at::Tensor& sin,
                  int64_t n_heads, int64_t D, int64_t rot, bool backward);
at::Tensor qk_norm_rope_fwd(const at::Tensor& x, at::Tensor& out, const at::Tensor& nw, const c10::optional<at::Tensor>& pos,
                            const at::Tensor& cos, const at::Tensor& sin, int64_t n_heads, int64_t D, int64_t rot, double eps);
void qk_norm_rope_bwd(const at::Tensor& dout, const at::Tensor& x, const at::Tensor& nw, const at::Tensor& rstd,
                      at::Tensor& dx, at::Tensor& dnw, const c10::optional<at::Tensor>& pos, const at::Tensor& cos,
                      const at::Tensor& sin, int64_t n_heads, int64_t D, int64_t rot);
void cross_entropy(at::Tensor& logits, const at::Tensor& labels, at::Tensor& loss, at::Tensor& stat_max,
                   at::Tensor& stat_sum, at::Tensor& stat_label, const at::Tensor& grad_scale, int64_t vocab_start,
                   int64_t ignore_index, int64_t mode, bool write_grad);
at::Tensor embedding_fwd(const at::Tensor& ids, const at::Tensor& W, int64_t vocab_start);
void embedding_bwd(const at::Tensor& ids, const at::Tensor& dout, at::Tensor& grad, int64_t vocab_start);
void adamw_step(at::Tensor& p, at::Tensor& m, at::Tensor& v, const at::Tensor& g, const c10::optional<at::Tensor>& p16,
                const at::Tensor& scalars, double beta1, double beta2, double eps, double wd);
int64_t sq_norm_scratch_elems();
void sq_norm_accum(const at::Tensor& x, at::Tensor& out, at::Tensor& scratch);
void cast_scale(const at::Tensor& src, at::Tensor& dst, double scale, bool accumulate);

}  // namespace pfb

TORCH_LIBRARY(pfb200, m) {
  m.def("read_status(bool reset) -> int", &pfb::op_read_status);
  m.def("set_wait_budget(float seconds) -> ()", &pfb::op_set_wait_budget);
  m.def("launch_count(bool reset) -> int", &pfb::op_launch_count);
  m.def("read_drop_count(bool reset) -> int", &pfb::op_read_drop_count);
  m.def("gemm(Tensor a, Tensor b, Tensor(a!) out, bool a_mn, bool b_mn, int epi, Tensor? out2, Tensor? block_expert, "
        "int n_per_expert, int force_bn) -> ()", &pfb::gemm);
  m.def("gemm_wgrad_grouped(Tensor dy, Tensor x, Tensor(a!) out, Tensor expert_rows) -> ()", &pfb::gemm_wgrad_grouped);
  m.def("attn_fwd(Tensor q, Tensor k, Tensor v, Tensor(a!) out, int B, int S, float scale, bool causal, Tensor? kend, "
        "Tensor? tile_min, Tensor? tile_max, bool p_in_tmem) -> Tensor", &pfb::attn_fwd);
  m.def("rms_norm_fwd(Tensor x, Tensor? residual, Tensor w, float eps) -> (Tensor, Tensor, Tensor)", &pfb::rms_norm_fwd);
  m.def("rms_norm_bwd_scratch_rows() -> int", &pfb::rms_norm_bwd_scratch_rows);
  m.def("rms_norm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd, Tensor? dres, Tensor(a!) dw_out, bool accumulate, "
        "Tensor(b!) scratch) -> Tensor", &pfb::rms_norm_bwd);
  m.def("swiglu_fwd(Tensor gu) -> Tensor", &pfb::swiglu_fwd);
  m.def("swiglu_bwd(Tensor dact, Tensor gu, bool want_act) -> (Tensor, Tensor)", &pfb::swiglu_bwd);
  m.def("rope_inplace(Tensor(a!) x, Tensor? pos, Tensor cos, Tensor sin, int n_heads, int D, int rot, bool backward) -> ()",
        &pfb::rope_inplace);
  m.def("qk_norm_rope_fwd(Tensor x, Tensor(a!) out, Tensor nw, Tensor? pos, Tensor cos, Tensor sin, int n_heads, int D, "
        "int rot, float eps) -> Tensor", &pfb::qk_norm_rope_fwd);
  m.def("qk_norm_rope_bwd(Tensor dout, Tensor x, Tensor nw, Tensor rstd, Tensor(a!) dx, Tensor(b!) dnw, Tensor? pos, "
        "Tensor cos, Tensor sin, int n_heads, int D, int rot) -> ()", &pfb::qk_norm_rope_bwd);
  m.def("cross_entropy(Tensor(a!) logits, Tensor labels, Tensor(b!) loss, Tensor(c!) stat_max, Tensor(d!) stat_sum, "
        "Tensor(e!) stat_label, Tensor grad_scale, int vocab_start, int ignore_index, int mode, bool write_grad) -> ()",
        &pfb::cross_entropy);
  m.def("embedding_fwd(Tensor ids, Tensor W, int vocab_start) -> Tensor", &pfb::embedding_fwd);
  m.def("embedding_bwd(Tensor ids, Tensor dout, Tensor(a!) grad, int vocab_start) -> ()", &pfb::embedding_bwd);
  m.def("adamw_step(Tensor(a!) p, Tensor(b!) m, Tensor(c!) v, Tensor g, Tensor? p16, Tensor scalars, float beta1, "
        "float beta2, float eps, float wd) -> ()", &pfb::adamw_step);
  m.def("sq_norm_scratch_elems() -> int", &pfb::sq_norm_scratch_elems);
  m.def("sq_norm_accum(Tensor x, Tensor(a!) out, Tensor(b!) scratch) -> ()", &pfb::sq_norm_accum);
  m.def("cast_scale(Tensor src, Tensor(a!) dst, float scale, bool accumulate) -> ()", &pfb::cast_scale);
}
