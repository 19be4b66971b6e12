// Operator registration: every kernel is reachable as torch.ops.q38.<name>.
#include <torch/extension.h>
#include <torch/library.h>

#include "host.h"

namespace q38 { std::atomic<long long> g_launches{0}; }

TORCH_LIBRARY(q38, m) {
  m.def("launch_count() -> int", []() -> int64_t { return (int64_t)q38::g_launches.load(); });
  m.def("gemm_bf16(Tensor a, Tensor b, Tensor(a!) c, bool a_mn_major, bool b_mn_major, float alpha, bool accumulate, Tensor(b!) err) -> ()");
  m.def("rmsnorm_fwd(Tensor x, Tensor w, float eps, bool out_bf16) -> Tensor[]");
  m.def("rmsnorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd) -> Tensor[]");
  m.def("gated_rmsnorm_fwd(Tensor x, Tensor gate, Tensor w, float eps) -> Tensor");
  m.def("gated_rmsnorm_bwd(Tensor dy, Tensor x, Tensor gate, Tensor w, float eps) -> Tensor[]");
  m.def("adamw_flat(Tensor(a!) p, Tensor g, Tensor(b!) m, Tensor(c!) v, Tensor? shadow, Tensor? grad_scale, int step, float lr, float wd, float beta1, float beta2, float eps) -> ()");
  m.def("sum_squares(Tensor x) -> Tensor");
}

TORCH_LIBRARY_IMPL(q38, CUDA, m) {
  m.impl("gemm_bf16", [](const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool amn, bool bmn, double alpha, bool acc, at::Tensor& err) {
    q38::gemm_bf16(a, b, c, amn, bmn, alpha, acc, err);
  });
  m.impl("rmsnorm_fwd", &q38::rmsnorm_fwd);
  m.impl("rmsnorm_bwd", &q38::rmsnorm_bwd);
  m.impl("gated_rmsnorm_fwd", &q38::gated_rmsnorm_fwd);
  m.impl("gated_rmsnorm_bwd", &q38::gated_rmsnorm_bwd);
  m.impl("adamw_flat", [](at::Tensor& p, const at::Tensor& g, at::Tensor& mm, at::Tensor& v, c10::optional<at::Tensor> shadow,
                          c10::optional<at::Tensor> gs, int64_t step, double lr, double wd, double b1, double b2, double eps) {
    q38::adamw_flat(p, g, mm, v, shadow, gs, step, lr, wd, b1, b2, eps);
  });
  m.impl("sum_squares", &q38::sum_squares);
}
