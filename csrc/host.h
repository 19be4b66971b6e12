// Host-side declarations shared by the extension's translation units.
#pragma once
#include <torch/extension.h>
#include <cuda.h>

#include <atomic>

namespace q38 {

// Number of kernels launched by this library since load (read by the benchmark).
extern std::atomic<long long> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

CUtensorMap make_tmap_bf16(const void* base, int64_t inner, int64_t rows, int64_t batch, int64_t row_stride_elems,
                           int64_t batch_stride_elems, int box_rows);

// gemm.cu
void gemm_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn_major, bool b_mn_major, double alpha,
               bool accumulate, at::Tensor& err);

// elementwise.cu
std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps, bool out_bf16);
std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd);
at::Tensor gated_rmsnorm_fwd(const at::Tensor& x, const at::Tensor& gate, const at::Tensor& w, double eps);
std::vector<at::Tensor> gated_rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& gate, const at::Tensor& w, double eps);
void adamw_flat(at::Tensor& p, const at::Tensor& g, at::Tensor& m, at::Tensor& v, c10::optional<at::Tensor> shadow,
                c10::optional<at::Tensor> grad_scale, int64_t step, double lr, double wd, double beta1, double beta2, double eps);
at::Tensor sum_squares(const at::Tensor& x);

}  // namespace q38
