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
CUtensorMap make_tmap_box(const void* base, int elem_bytes, int64_t inner, int64_t rows, int64_t batch, int64_t row_stride_elems,
                          int64_t batch_stride_elems, int box_rows, int box_inner_bytes);

// gemm.cu
void gemm_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn_major, bool b_mn_major, double alpha,
               bool accumulate, at::Tensor& err, int64_t splits);

void gemm_bf16_persistent(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn_major, bool b_mn_major, double alpha,
                          bool accumulate, at::Tensor& err, int64_t splits, const c10::optional<at::Tensor>& addend = c10::nullopt, double beta = 0.0);

// mxfp8.cu
int64_t mxfp8_pick_bn(int64_t N);
std::vector<at::Tensor> mxfp8_quantize_rows(const at::Tensor& src, const c10::optional<at::Tensor>& perm, int64_t topk, const at::Tensor& sched, int64_t P);
std::vector<at::Tensor> mxfp8_quantize_weight(const at::Tensor& w, int64_t bn);
void mxfp8_grouped_gemm(const at::Tensor& aq, const at::Tensor& sfa, const at::Tensor& wq, const at::Tensor& sfw, at::Tensor& out, const at::Tensor& sched, int64_t bn,
                        at::Tensor& err);

// muon.cu
void muon_prepass(const at::Tensor& grads, at::Tensor& buf, at::Tensor& work, at::Tensor& sumsq, const at::Tensor& mats, const at::Tensor& tiles,
                  const c10::optional<at::Tensor>& grad_scale, double momentum, const c10::optional<at::Tensor>& err);
void muon_normalize(at::Tensor& work, at::Tensor& sumsq, const at::Tensor& mats, const at::Tensor& tiles, double eps, const c10::optional<at::Tensor>& err);
void muon_apply(at::Tensor& params, const c10::optional<at::Tensor>& shadow, const at::Tensor& work, const at::Tensor& mats, const at::Tensor& tiles,
                const at::Tensor& scales, const c10::optional<at::Tensor>& hyper, double lr, double wd, const c10::optional<at::Tensor>& err);
void muon_small_ns(const at::Tensor& src, at::Tensor& dst, int64_t rows, int64_t cols, int64_t steps, const c10::optional<at::Tensor>& err);

// qsa_prep.cu
std::vector<at::Tensor> qsa_headprep_fwd(const at::Tensor& src, const c10::optional<at::Tensor>& w, const at::Tensor& cosv, const at::Tensor& sinv, double eps,
                                         bool split_gate);
std::vector<at::Tensor> qsa_headprep_bwd(const at::Tensor& dout, const c10::optional<at::Tensor>& dgate, const at::Tensor& src, const c10::optional<at::Tensor>& w,
                                         const at::Tensor& cosv, const at::Tensor& sinv, const at::Tensor& rstd);

at::Tensor gate_add_fwd(const at::Tensor& routed, const at::Tensor& shared, const at::Tensor& logit);
std::vector<at::Tensor> gate_add_bwd(const at::Tensor& dy, const at::Tensor& shared, const at::Tensor& logit);

std::vector<at::Tensor> gdn_gates_fwd(const at::Tensor& b_raw, const at::Tensor& a_raw, const at::Tensor& A_log, const at::Tensor& dt_bias);
std::vector<at::Tensor> gdn_gates_bwd(const at::Tensor& dbeta, const at::Tensor& dg, const at::Tensor& b_raw, const at::Tensor& a_raw, const at::Tensor& A_log,
                                      const at::Tensor& dt_bias);

at::Tensor swiglu_fwd(const at::Tensor& g, const at::Tensor& u);
std::vector<at::Tensor> swiglu_bwd(const at::Tensor& dy, const at::Tensor& g, const at::Tensor& u);

at::Tensor sigmoid_mul_fwd(const at::Tensor& x, const at::Tensor& g);
std::vector<at::Tensor> sigmoid_mul_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& g);

// ngram.cu
void embed_bwd(const at::Tensor& ids, const at::Tensor& dout, at::Tensor& grad);
std::vector<at::Tensor> ngram_fwd(const at::Tensor& ids, const at::Tensor& emb2, const at::Tensor& emb3, const at::Tensor& norm_w, int64_t vocab,
                                  int64_t eos, double eps);
at::Tensor ngram_bwd(const at::Tensor& de, const at::Tensor& rows, const at::Tensor& emb2, const at::Tensor& emb3, const at::Tensor& norm_w,
                     const at::Tensor& rstd, at::Tensor& g2, at::Tensor& g3);

// elementwise.cu
std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps, bool out_bf16);
std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd);
at::Tensor gated_rmsnorm_fwd(const at::Tensor& x, const at::Tensor& gate, const at::Tensor& w, double eps);
std::vector<at::Tensor> gated_rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& gate, const at::Tensor& w, double eps);
void adamw_flat(at::Tensor& p, const at::Tensor& g, at::Tensor& m, at::Tensor& v, c10::optional<at::Tensor> shadow,
                c10::optional<at::Tensor> grad_scale, int64_t step, double lr, double wd, double beta1, double beta2, double eps,
                c10::optional<at::Tensor> hyper, c10::optional<at::Tensor> err = c10::nullopt);
at::Tensor sum_squares(const at::Tensor& x);

// mhc.cu
std::vector<at::Tensor> mhc_coef_fwd(const at::Tensor& X, const at::Tensor& Lraw, const at::Tensor& Bw, const at::Tensor& b_pre,
                                     const at::Tensor& b_post, const at::Tensor& b_res, const at::Tensor& alphas, const at::Tensor& norm_w,
                                     int64_t iters, double norm_eps, bool out_bf16);
at::Tensor mhc_post_fwd(const at::Tensor& X, const at::Tensor& y, const at::Tensor& coef);
std::vector<at::Tensor> mhc_post_bwd(const at::Tensor& dXo, const at::Tensor& X, const at::Tensor& y, const at::Tensor& coef);
std::vector<at::Tensor> mhc_pre_bwd_a(const at::Tensor& dxout, const at::Tensor& X, const at::Tensor& Lraw, const at::Tensor& Bw,
                                      const at::Tensor& b_pre, const at::Tensor& b_post, const at::Tensor& b_res, const at::Tensor& alphas,
                                      const at::Tensor& norm_w, const at::Tensor& coef, const at::Tensor& z, const at::Tensor& inv,
                                      const at::Tensor& rstd, at::Tensor& dcoef, int64_t iters);
at::Tensor mhc_pre_bwd_c(const at::Tensor& G, const at::Tensor& dXo, const at::Tensor& X, const at::Tensor& dxin, const at::Tensor& coef, const at::Tensor& c1);

// moe.cu
std::vector<at::Tensor> moe_route_fwd(const at::Tensor& logits, int64_t k);
at::Tensor moe_route_bwd(const at::Tensor& probs, const at::Tensor& top_idx, const at::Tensor& top_w, const at::Tensor& d_top_w,
                         const c10::optional<at::Tensor>& d_prob_sum);
std::vector<at::Tensor> moe_sort(const at::Tensor& top_idx, int64_t E, const c10::optional<at::Tensor>& err = c10::nullopt);
at::Tensor moe_gather(const at::Tensor& x, const at::Tensor& perm, int64_t k);
at::Tensor moe_combine_fwd(const at::Tensor& y_sorted, const at::Tensor& inv_perm, const at::Tensor& top_w);
std::vector<at::Tensor> moe_combine_bwd(const at::Tensor& dout, const at::Tensor& y_sorted, const at::Tensor& inv_perm, const at::Tensor& top_w);
at::Tensor moe_unpermute_sum(const at::Tensor& dx_sorted, const at::Tensor& inv_perm, int64_t T, int64_t k);
void moe_grouped_gemm(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& out, const at::Tensor& sched, bool b_mn_major, at::Tensor& err);
void moe_grouped_swiglu(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& hmid, at::Tensor& gu, const at::Tensor& sched, at::Tensor& err);
void moe_grouped_dswiglu(const at::Tensor& dy, const at::Tensor& w_down, const at::Tensor& gu, at::Tensor& dgu, const at::Tensor& sched, at::Tensor& err);
void moe_grouped_wgrad(const at::Tensor& a, const at::Tensor& b, at::Tensor& grad, const at::Tensor& offsets, at::Tensor& err);

// moe_persistent.cu
bool moe_persistent_enabled();
void moe_set_persistent(int64_t mode);
void moe_grouped_gemm_p(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& out, const at::Tensor& sched, bool b_mn_major, at::Tensor& err);
void moe_grouped_swiglu_p(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& hmid, at::Tensor& gu, const at::Tensor& sched, at::Tensor& err);
void moe_grouped_dswiglu_p(const at::Tensor& dy, const at::Tensor& w_down, const at::Tensor& gu, at::Tensor& dgu, const at::Tensor& sched, at::Tensor& err);

// gdn.cu
std::vector<at::Tensor> gdn_scan_fwd(const at::Tensor& w, const at::Tensor& u, const at::Tensor& P, const at::Tensor& qg, const at::Tensor& kg,
                                     const at::Tensor& dch, int64_t B, int64_t H);
std::vector<at::Tensor> gdn_scan_bwd(const at::Tensor& w, const at::Tensor& P, const at::Tensor& qg, const at::Tensor& kg, const at::Tensor& dch,
                                     const at::Tensor& vnew, const at::Tensor& states, const at::Tensor& dout, int64_t B, int64_t H);

std::vector<at::Tensor> gdn_prep_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g, const at::Tensor& beta);
std::vector<at::Tensor> gdn_prep_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g, const at::Tensor& beta,
                                     const at::Tensor& Tm, const at::Tensor& dw, const at::Tensor& du, const at::Tensor& dP, const at::Tensor& dqg,
                                     const at::Tensor& dkg, const at::Tensor& dd);
// qsa_index.cu
at::Tensor qsa_main_block_stats(const at::Tensor& q, const at::Tensor& k, double scale);
at::Tensor qsa_indexer_fwd(const at::Tensor& qi, const at::Tensor& ki, const at::Tensor& wi, double scale);
std::vector<at::Tensor> qsa_kl_combine(const c10::optional<at::Tensor>& stats, const at::Tensor& blse, int64_t nq);
std::vector<at::Tensor> qsa_select(const at::Tensor& lp_blk, int64_t budget);
std::vector<at::Tensor> qsa_indexer_bwd(const at::Tensor& qi, const at::Tensor& ki, const at::Tensor& wi, const at::Tensor& blse, const at::Tensor& dblse,
                                        double gscale, double scale);
// qsa_tc.cu
at::Tensor qsa_block_stats_tc(const at::Tensor& q, const at::Tensor& k, double scale, at::Tensor& err);
// qsa_attn.cu
std::vector<at::Tensor> qsa_attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const c10::optional<at::Tensor>& count,
                                     const c10::optional<at::Tensor>& index, double scale);
std::vector<at::Tensor> qsa_attn_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o, const at::Tensor& dout,
                                     const at::Tensor& lse, const at::Tensor& sel, double scale);
// ep.cu
void ep_publish_counts(const at::Tensor& offsets, int64_t rank, std::vector<int64_t> peer_counts);
std::vector<at::Tensor> ep_plan(const at::Tensor& counts_all, int64_t rank, int64_t world, int64_t capacity, at::Tensor& err);
void ep_dispatch(const at::Tensor& src, const at::Tensor& perm, const at::Tensor& expert_of_pair, const at::Tensor& offsets, const at::Tensor& send_base,
                 int64_t K, int64_t E_loc, int64_t capacity, bool gather, int64_t rank, std::vector<int64_t> recv_rows, std::vector<int64_t> ret_rank,
                 std::vector<int64_t> ret_row);
void moe_grouped_gemm_return(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& out, const at::Tensor& sched, bool b_mn_major, at::Tensor& err,
                             const at::Tensor& ret_rank, const at::Tensor& ret_row, std::vector<int64_t> peer_out);
// comm.cu
at::Tensor p2p_alloc(int64_t nbytes, int64_t device);
at::Tensor p2p_get_handle(const at::Tensor& t);
int64_t p2p_open_handle(const at::Tensor& handle, int64_t device);
void p2p_close_handle(int64_t ptr, int64_t device);
void p2p_barrier(at::Tensor& own_flags, std::vector<int64_t> peer_flags, int64_t rank, int64_t epoch, double wait_seconds, at::Tensor& err);
void p2p_reduce_scatter(std::vector<int64_t> grads, int64_t rank, int64_t start, int64_t count, double scale, int64_t device,
                        const c10::optional<at::Tensor>& err);
void p2p_all_gather(const at::Tensor& params, const c10::optional<at::Tensor>& shadow, std::vector<int64_t> peer_params, std::vector<int64_t> peer_shadow,
                    int64_t rank, int64_t start, int64_t count, const c10::optional<at::Tensor>& err);
void nvls_reduce_scatter(int64_t mc_grads, at::Tensor& grads, int64_t start, int64_t count, double scale, const c10::optional<at::Tensor>& err);
void nvls_all_gather(const at::Tensor& params, int64_t mc_params, int64_t start, int64_t count, const c10::optional<at::Tensor>& err);
void p2p_push_segments(const at::Tensor& grads, std::vector<int64_t> peer_staging, std::vector<int64_t> starts, std::vector<int64_t> counts, int64_t slot_stride,
                       int64_t rank, const c10::optional<at::Tensor>& err);
void p2p_reduce_staged(at::Tensor& grads, const at::Tensor& staging, int64_t slot_stride, int64_t rank, int64_t world, int64_t start, int64_t count, double scale,
                       const c10::optional<at::Tensor>& err);
void cast_shadow_except(const at::Tensor& params, at::Tensor& shadow, int64_t skip_start, int64_t skip_count, const c10::optional<at::Tensor>& err);
void p2p_publish_scalar(const at::Tensor& value, std::vector<int64_t> peer_slots, int64_t rank);
// ce.cu
at::Tensor ce_inplace(at::Tensor& logits, const at::Tensor& target);
// conv.cu
at::Tensor conv_silu_fwd(const at::Tensor& x, const at::Tensor& w);
std::vector<at::Tensor> conv_silu_bwd(const at::Tensor& x, const at::Tensor& w, const at::Tensor& dy);

}  // namespace q38
