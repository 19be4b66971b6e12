// Operator registration: every kernel is reachable as torch.ops.q38.<name>.
#include <torch/extension.h>
#include <torch/library.h>

#include "host.h"

namespace q38 {
std::atomic<long long> g_launches{0};
at::Tensor qsa_first_query_lp(const at::Tensor& q_first, const at::Tensor& ki, const at::Tensor& w_first, double scale);   // qsa_first.cu
bool gemm_bf16_pair(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, double alpha, bool accumulate, at::Tensor& err);   // gemm_pair.cu
}

TORCH_LIBRARY(q38, m) {
  m.def("launch_count() -> int", []() -> int64_t { return (int64_t)q38::g_launches.load(); });
  m.def("gemm_bf16(Tensor a, Tensor b, Tensor(a!) c, bool a_mn_major, bool b_mn_major, float alpha, bool accumulate, Tensor(b!) err, int splits) -> ()");
  m.def("gemm_bf16_persistent(Tensor a, Tensor b, Tensor(a!) c, bool a_mn_major, bool b_mn_major, float alpha, bool accumulate, Tensor(b!) err, int splits, Tensor? addend=None, float beta=0.0) -> ()",
        [](const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool amn, bool bmn, double alpha, bool acc, at::Tensor& err, int64_t splits,
           c10::optional<at::Tensor> addend, double beta) {
          q38::gemm_bf16_persistent(a, b, c, amn, bmn, alpha, acc, err, splits, addend, beta);
        });
  m.def("mxfp8_pick_bn(int N) -> int", &q38::mxfp8_pick_bn);
  m.def("mxfp8_quantize_rows(Tensor src, Tensor? perm, int topk, Tensor sched, int P) -> Tensor[]",
        [](const at::Tensor& src, c10::optional<at::Tensor> perm, int64_t topk, const at::Tensor& sched, int64_t P) { return q38::mxfp8_quantize_rows(src, perm, topk, sched, P); });
  m.def("mxfp8_quantize_weight(Tensor w, int bn) -> Tensor[]", &q38::mxfp8_quantize_weight);
  m.def("mxfp8_grouped_gemm(Tensor aq, Tensor sfa, Tensor wq, Tensor sfw, Tensor(a!) out, Tensor sched, int bn, Tensor(b!) err) -> ()",
        [](const at::Tensor& aq, const at::Tensor& sfa, const at::Tensor& wq, const at::Tensor& sfw, at::Tensor& out, const at::Tensor& sched, int64_t bn, at::Tensor& err) {
          q38::mxfp8_grouped_gemm(aq, sfa, wq, sfw, out, sched, bn, err);
        });
  m.def("muon_prepass(Tensor grads, Tensor(a!) buf, Tensor(b!) work, Tensor(c!) sumsq, Tensor mats, Tensor tiles, Tensor? grad_scale, float momentum, Tensor? err) -> ()",
        [](const at::Tensor& g, at::Tensor& b, at::Tensor& w, at::Tensor& s, const at::Tensor& mats, const at::Tensor& tiles, c10::optional<at::Tensor> gs, double mom,
           c10::optional<at::Tensor> err) { q38::muon_prepass(g, b, w, s, mats, tiles, gs, mom, err); });
  m.def("muon_normalize(Tensor(a!) work, Tensor(b!) sumsq, Tensor mats, Tensor tiles, float eps, Tensor? err) -> ()",
        [](at::Tensor& w, at::Tensor& s, const at::Tensor& mats, const at::Tensor& tiles, double eps, c10::optional<at::Tensor> err) {
          q38::muon_normalize(w, s, mats, tiles, eps, err);
        });
  m.def("muon_apply(Tensor(a!) params, Tensor? shadow, Tensor work, Tensor mats, Tensor tiles, Tensor scales, Tensor? hyper, float lr, float wd, Tensor? err) -> ()",
        [](at::Tensor& p, c10::optional<at::Tensor> sh, const at::Tensor& w, const at::Tensor& mats, const at::Tensor& tiles, const at::Tensor& scales,
           c10::optional<at::Tensor> hyper, double lr, double wd, c10::optional<at::Tensor> err) { q38::muon_apply(p, sh, w, mats, tiles, scales, hyper, lr, wd, err); });
  m.def("muon_small_ns(Tensor src, Tensor(a!) dst, int rows, int cols, int steps, Tensor? err) -> ()",
        [](const at::Tensor& src, at::Tensor& dst, int64_t rows, int64_t cols, int64_t steps, c10::optional<at::Tensor> err) {
          q38::muon_small_ns(src, dst, rows, cols, steps, err);
        });
  m.def("cast_shadow_except(Tensor params, Tensor(a!) shadow, int skip_start, int skip_count, Tensor? err) -> ()",
        [](const at::Tensor& p, at::Tensor& sh, int64_t s0, int64_t n, c10::optional<at::Tensor> err) { q38::cast_shadow_except(p, sh, s0, n, err); });
  m.def("qsa_headprep_fwd(Tensor src, Tensor? w, Tensor cos, Tensor sin, float eps, bool split_gate) -> Tensor[]", &q38::qsa_headprep_fwd);
  m.def("qsa_headprep_bwd(Tensor dout, Tensor? dgate, Tensor src, Tensor? w, Tensor cos, Tensor sin, Tensor rstd) -> Tensor[]", &q38::qsa_headprep_bwd);
  m.def("gate_add_fwd(Tensor routed, Tensor shared, Tensor logit) -> Tensor", &q38::gate_add_fwd);
  m.def("gate_add_bwd(Tensor dy, Tensor shared, Tensor logit) -> Tensor[]", &q38::gate_add_bwd);
  m.def("gdn_gates_fwd(Tensor b_raw, Tensor a_raw, Tensor A_log, Tensor dt_bias) -> Tensor[]", &q38::gdn_gates_fwd);
  m.def("gdn_gates_bwd(Tensor dbeta, Tensor dg, Tensor b_raw, Tensor a_raw, Tensor A_log, Tensor dt_bias) -> Tensor[]", &q38::gdn_gates_bwd);
  m.def("embed_bwd(Tensor ids, Tensor dout, Tensor(a!) grad) -> ()", &q38::embed_bwd);
  m.def("swiglu_fwd(Tensor g, Tensor u) -> Tensor", &q38::swiglu_fwd);
  m.def("swiglu_bwd(Tensor dy, Tensor g, Tensor u) -> Tensor[]", &q38::swiglu_bwd);
  m.def("sigmoid_mul_fwd(Tensor x, Tensor g) -> Tensor", &q38::sigmoid_mul_fwd);
  m.def("sigmoid_mul_bwd(Tensor dy, Tensor x, Tensor g) -> Tensor[]", &q38::sigmoid_mul_bwd);
  m.def("ngram_fwd(Tensor ids, Tensor emb2, Tensor emb3, Tensor norm_w, int vocab, int eos, float eps) -> Tensor[]", &q38::ngram_fwd);
  m.def("ngram_bwd(Tensor de, Tensor rows, Tensor emb2, Tensor emb3, Tensor norm_w, Tensor rstd, Tensor(a!) g2, Tensor(b!) g3) -> Tensor", &q38::ngram_bwd);
  m.def("rmsnorm_fwd(Tensor x, Tensor w, float eps, bool out_bf16) -> Tensor[]");
  m.def("rmsnorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd) -> Tensor[]");
  m.def("gated_rmsnorm_fwd(Tensor x, Tensor gate, Tensor w, float eps) -> Tensor");
  m.def("gated_rmsnorm_bwd(Tensor dy, Tensor x, Tensor gate, Tensor w, float eps) -> Tensor[]");
  m.def("adamw_flat(Tensor(a!) p, Tensor g, Tensor(b!) m, Tensor(c!) v, Tensor? shadow, Tensor? grad_scale, int step, float lr, float wd, float beta1, float beta2, float eps, Tensor? hyper, Tensor? err=None) -> ()");
  m.def("sum_squares(Tensor x) -> Tensor");
  m.def("qsa_main_block_stats(Tensor q, Tensor k, float scale) -> Tensor");
  m.def("qsa_block_stats_tc(Tensor q, Tensor k, float scale, Tensor(a!) err) -> Tensor",
        [](const at::Tensor& q, const at::Tensor& k, double scale, at::Tensor& err) { return q38::qsa_block_stats_tc(q, k, scale, err); });
  m.def("qsa_indexer_fwd(Tensor qi, Tensor ki, Tensor wi, float scale) -> Tensor");
  m.def("gemm_pair(Tensor a, Tensor b, Tensor(a!) c, float alpha, bool accumulate, Tensor(b!) err) -> bool",
        [](const at::Tensor& a, const at::Tensor& b, at::Tensor& c, double alpha, bool acc, at::Tensor& err) { return q38::gemm_bf16_pair(a, b, c, alpha, acc, err); });
  m.def("qsa_first_query_lp(Tensor q_first, Tensor ki, Tensor w_first, float scale) -> Tensor", &q38::qsa_first_query_lp);
  m.def("qsa_kl_combine(Tensor? stats, Tensor blse, int nq) -> Tensor[]");
  m.def("qsa_select(Tensor lp_blk, int budget) -> Tensor[]");
  m.def("qsa_indexer_bwd(Tensor qi, Tensor ki, Tensor wi, Tensor blse, Tensor dblse, float gscale, float scale) -> Tensor[]");
  m.def("qsa_attn_fwd(Tensor q, Tensor k, Tensor v, Tensor? count, Tensor? index, float scale) -> Tensor[]");
  m.def("qsa_attn_bwd(Tensor q, Tensor k, Tensor v, Tensor o, Tensor dout, Tensor lse, Tensor sel, float scale) -> Tensor[]");
  m.def("ep_publish_counts(Tensor offsets, int rank, int[] peer_counts) -> ()",
        [](const at::Tensor& o, int64_t rank, std::vector<int64_t> peers) { q38::ep_publish_counts(o, rank, peers); });
  m.def("ep_plan(Tensor counts_all, int rank, int world, int capacity, Tensor(a!) err) -> Tensor[]",
        [](const at::Tensor& c, int64_t rank, int64_t world, int64_t cap, at::Tensor& err) { return q38::ep_plan(c, rank, world, cap, err); });
  m.def("ep_dispatch(Tensor src, Tensor perm, Tensor expert_of_pair, Tensor offsets, Tensor send_base, int K, int E_loc, int capacity, bool gather, int rank, int[] recv_rows, int[] ret_rank, int[] ret_row) -> ()",
        [](const at::Tensor& a, const at::Tensor& b, const at::Tensor& c, const at::Tensor& d, const at::Tensor& e, int64_t K, int64_t El, int64_t cap, bool g, int64_t rank,
           std::vector<int64_t> r0, std::vector<int64_t> r1, std::vector<int64_t> r2) { q38::ep_dispatch(a, b, c, d, e, K, El, cap, g, rank, r0, r1, r2); });
  m.def("moe_grouped_gemm_return(Tensor rows, Tensor weight, Tensor out, Tensor sched, bool b_mn_major, Tensor(a!) err, Tensor ret_rank, Tensor ret_row, int[] peer_out) -> ()",
        [](const at::Tensor& r, const at::Tensor& w, at::Tensor o, const at::Tensor& s, bool mn, at::Tensor& err, const at::Tensor& rr, const at::Tensor& rw, std::vector<int64_t> po) {
          q38::moe_grouped_gemm_return(r, w, o, s, mn, err, rr, rw, po);
        });
  m.def("p2p_alloc(int nbytes, int device) -> Tensor", &q38::p2p_alloc);
  m.def("p2p_get_handle(Tensor t) -> Tensor", &q38::p2p_get_handle);
  m.def("p2p_open_handle(Tensor handle, int device) -> int", &q38::p2p_open_handle);
  m.def("p2p_close_handle(int ptr, int device) -> ()", &q38::p2p_close_handle);
  m.def("p2p_barrier(Tensor(a!) own_flags, int[] peer_flags, int rank, int epoch, float wait_seconds, Tensor(b!) err) -> ()",
        [](at::Tensor& f, std::vector<int64_t> peers, int64_t rank, int64_t epoch, double wait, at::Tensor& err) { q38::p2p_barrier(f, peers, rank, epoch, wait, err); });
  m.def("p2p_reduce_scatter(int[] grads, int rank, int start, int count, float scale, int device, Tensor? err=None) -> ()",
        [](std::vector<int64_t> g, int64_t rank, int64_t start, int64_t count, double scale, int64_t dev, c10::optional<at::Tensor> err) {
          q38::p2p_reduce_scatter(g, rank, start, count, scale, dev, err);
        });
  m.def("p2p_all_gather(Tensor params, Tensor? shadow, int[] peer_params, int[] peer_shadow, int rank, int start, int count, Tensor? err=None) -> ()",
        [](const at::Tensor& p, c10::optional<at::Tensor> sh, std::vector<int64_t> pp, std::vector<int64_t> ps, int64_t rank, int64_t start, int64_t count,
           c10::optional<at::Tensor> err) { q38::p2p_all_gather(p, sh, pp, ps, rank, start, count, err); });
  m.def("nvls_reduce_scatter(int mc_grads, Tensor(a!) grads, int start, int count, float scale, Tensor? err=None) -> ()",
        [](int64_t mc, at::Tensor& g, int64_t start, int64_t count, double scale, c10::optional<at::Tensor> err) { q38::nvls_reduce_scatter(mc, g, start, count, scale, err); });
  m.def("nvls_all_gather(Tensor params, int mc_params, int start, int count, Tensor? err=None) -> ()",
        [](const at::Tensor& p, int64_t mc, int64_t start, int64_t count, c10::optional<at::Tensor> err) { q38::nvls_all_gather(p, mc, start, count, err); });
  m.def("p2p_push_segments(Tensor grads, int[] peer_staging, int[] starts, int[] counts, int slot_stride, int rank, Tensor? err=None) -> ()",
        [](const at::Tensor& g, std::vector<int64_t> st, std::vector<int64_t> starts, std::vector<int64_t> counts, int64_t stride, int64_t rank,
           c10::optional<at::Tensor> err) { q38::p2p_push_segments(g, st, starts, counts, stride, rank, err); });
  m.def("p2p_reduce_staged(Tensor(a!) grads, Tensor staging, int slot_stride, int rank, int world, int start, int count, float scale, Tensor? err=None) -> ()",
        [](at::Tensor& g, const at::Tensor& st, int64_t stride, int64_t rank, int64_t world, int64_t start, int64_t count, double scale, c10::optional<at::Tensor> err) {
          q38::p2p_reduce_staged(g, st, stride, rank, world, start, count, scale, err);
        });
  m.def("p2p_publish_scalar(Tensor value, int[] peer_slots, int rank) -> ()",
        [](const at::Tensor& v, std::vector<int64_t> slots, int64_t rank) { q38::p2p_publish_scalar(v, slots, rank); });
  m.def("moe_set_persistent(int mode) -> ()", [](int64_t mode) { q38::moe_set_persistent(mode); });
  m.def("ce_inplace(Tensor(a!) logits, Tensor target) -> Tensor", [](at::Tensor& l, const at::Tensor& t) { return q38::ce_inplace(l, t); });
  m.def("conv_silu_fwd(Tensor x, Tensor w) -> Tensor");
  m.def("conv_silu_bwd(Tensor x, Tensor w, Tensor dy) -> Tensor[]");
  m.def("gdn_prep_fwd(Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta) -> Tensor[]");
  m.def("gdn_prep_bwd(Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta, Tensor Tm, Tensor dw, Tensor du, Tensor dP, Tensor dqg, Tensor dkg, Tensor dd) -> Tensor[]");
  m.def("gdn_scan_fwd(Tensor w, Tensor u, Tensor P, Tensor qg, Tensor kg, Tensor dch, int B, int H) -> Tensor[]");
  m.def("gdn_scan_bwd(Tensor w, Tensor P, Tensor qg, Tensor kg, Tensor dch, Tensor vnew, Tensor states, Tensor dout, int B, int H) -> Tensor[]");
  m.def("moe_route_fwd(Tensor logits, int k) -> Tensor[]");
  m.def("moe_route_bwd(Tensor probs, Tensor top_idx, Tensor top_w, Tensor d_top_w, Tensor? d_prob_sum) -> Tensor");
  m.def("moe_sort(Tensor top_idx, int E, Tensor? err=None) -> Tensor[]");
  m.def("moe_gather(Tensor x, Tensor perm, int k) -> Tensor");
  m.def("moe_combine_fwd(Tensor y_sorted, Tensor inv_perm, Tensor top_w) -> Tensor");
  m.def("moe_combine_bwd(Tensor dout, Tensor y_sorted, Tensor inv_perm, Tensor top_w) -> Tensor[]");
  m.def("moe_unpermute_sum(Tensor dx_sorted, Tensor inv_perm, int T, int k) -> Tensor");
  m.def("moe_grouped_gemm(Tensor rows, Tensor weight, Tensor(a!) out, Tensor sched, bool b_mn_major, Tensor(b!) err) -> ()");
  m.def("moe_grouped_swiglu(Tensor rows, Tensor weight, Tensor(a!) hmid, Tensor(b!) gu, Tensor sched, Tensor(c!) err) -> ()");
  m.def("moe_grouped_dswiglu(Tensor dy, Tensor w_down, Tensor gu, Tensor(a!) dgu, Tensor sched, Tensor(b!) err) -> ()");
  m.def("moe_grouped_wgrad(Tensor a, Tensor b, Tensor(a!) grad, Tensor offsets, Tensor(b!) err) -> ()");
  m.def("mhc_coef_fwd(Tensor X, Tensor Lraw, Tensor Bw, Tensor b_pre, Tensor b_post, Tensor b_res, Tensor alphas, Tensor norm_w, int iters, float norm_eps, bool out_bf16) -> Tensor[]");
  m.def("mhc_post_fwd(Tensor X, Tensor y, Tensor coef) -> Tensor");
  m.def("mhc_post_bwd(Tensor dXo, Tensor X, Tensor y, Tensor coef) -> Tensor[]");
  m.def("mhc_pre_bwd_a(Tensor dxout, Tensor X, Tensor Lraw, Tensor Bw, Tensor b_pre, Tensor b_post, Tensor b_res, Tensor alphas, Tensor norm_w, Tensor coef, Tensor z, Tensor inv, Tensor rstd, Tensor(a!) dcoef, int iters) -> Tensor[]");
  m.def("mhc_pre_bwd_c(Tensor G, Tensor dXo, Tensor X, Tensor dxin, Tensor coef, Tensor c1) -> Tensor");
}

TORCH_LIBRARY_IMPL(q38, CUDA, m) {
  m.impl("gemm_bf16", [](const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool amn, bool bmn, double alpha, bool acc, at::Tensor& err, int64_t splits) {
    q38::gemm_bf16(a, b, c, amn, bmn, alpha, acc, err, splits);
  });
  m.impl("rmsnorm_fwd", &q38::rmsnorm_fwd);
  m.impl("rmsnorm_bwd", &q38::rmsnorm_bwd);
  m.impl("gated_rmsnorm_fwd", &q38::gated_rmsnorm_fwd);
  m.impl("gated_rmsnorm_bwd", &q38::gated_rmsnorm_bwd);
  m.impl("adamw_flat", [](at::Tensor& p, const at::Tensor& g, at::Tensor& mm, at::Tensor& v, c10::optional<at::Tensor> shadow,
                          c10::optional<at::Tensor> gs, int64_t step, double lr, double wd, double b1, double b2, double eps,
                          c10::optional<at::Tensor> hyper, c10::optional<at::Tensor> err) {
    q38::adamw_flat(p, g, mm, v, shadow, gs, step, lr, wd, b1, b2, eps, hyper, err);
  });
  m.impl("sum_squares", &q38::sum_squares);
  m.impl("qsa_main_block_stats", &q38::qsa_main_block_stats);
  m.impl("qsa_indexer_fwd", &q38::qsa_indexer_fwd);
  m.impl("qsa_kl_combine", [](c10::optional<at::Tensor> stats, const at::Tensor& blse, int64_t nq) { return q38::qsa_kl_combine(stats, blse, nq); });
  m.impl("qsa_select", &q38::qsa_select);
  m.impl("qsa_indexer_bwd", &q38::qsa_indexer_bwd);
  m.impl("qsa_attn_fwd", [](const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, c10::optional<at::Tensor> c, c10::optional<at::Tensor> i, double s) {
    return q38::qsa_attn_fwd(q, k, v, c, i, s);
  });
  m.impl("qsa_attn_bwd", &q38::qsa_attn_bwd);
  m.impl("conv_silu_fwd", &q38::conv_silu_fwd);
  m.impl("conv_silu_bwd", &q38::conv_silu_bwd);
  m.impl("gdn_prep_fwd", &q38::gdn_prep_fwd);
  m.impl("gdn_prep_bwd", &q38::gdn_prep_bwd);
  m.impl("gdn_scan_fwd", &q38::gdn_scan_fwd);
  m.impl("gdn_scan_bwd", &q38::gdn_scan_bwd);
  m.impl("moe_route_fwd", &q38::moe_route_fwd);
  m.impl("moe_route_bwd", [](const at::Tensor& a, const at::Tensor& b, const at::Tensor& c, const at::Tensor& d, c10::optional<at::Tensor> e) {
    return q38::moe_route_bwd(a, b, c, d, e);
  });
  m.impl("moe_sort", [](const at::Tensor& idx, int64_t E, c10::optional<at::Tensor> err) { return q38::moe_sort(idx, E, err); });
  m.impl("moe_gather", &q38::moe_gather);
  m.impl("moe_combine_fwd", &q38::moe_combine_fwd);
  m.impl("moe_combine_bwd", &q38::moe_combine_bwd);
  m.impl("moe_unpermute_sum", &q38::moe_unpermute_sum);
  m.impl("moe_grouped_gemm", [](const at::Tensor& a, const at::Tensor& b, at::Tensor& c, const at::Tensor& d, bool mn, at::Tensor& err) {
    q38::moe_grouped_gemm(a, b, c, d, mn, err);
  });
  m.impl("moe_grouped_swiglu", [](const at::Tensor& a, const at::Tensor& b, at::Tensor& c, at::Tensor& d, const at::Tensor& e, at::Tensor& err) {
    q38::moe_grouped_swiglu(a, b, c, d, e, err);
  });
  m.impl("moe_grouped_dswiglu", [](const at::Tensor& a, const at::Tensor& b, const at::Tensor& c, at::Tensor& d, const at::Tensor& e, at::Tensor& err) {
    q38::moe_grouped_dswiglu(a, b, c, d, e, err);
  });
  m.impl("moe_grouped_wgrad", [](const at::Tensor& a, const at::Tensor& b, at::Tensor& c, const at::Tensor& d, at::Tensor& err) {
    q38::moe_grouped_wgrad(a, b, c, d, err);
  });
  m.impl("mhc_coef_fwd", &q38::mhc_coef_fwd);
  m.impl("mhc_post_fwd", &q38::mhc_post_fwd);
  m.impl("mhc_post_bwd", &q38::mhc_post_bwd);
  m.impl("mhc_pre_bwd_a", [](const at::Tensor& a, const at::Tensor& b, const at::Tensor& c, const at::Tensor& d, const at::Tensor& e,
                             const at::Tensor& f, const at::Tensor& g, const at::Tensor& h, const at::Tensor& i, const at::Tensor& j,
                             const at::Tensor& k, const at::Tensor& l, const at::Tensor& mm, at::Tensor& n, int64_t it) {
    return q38::mhc_pre_bwd_a(a, b, c, d, e, f, g, h, i, j, k, l, mm, n, it);
  });
  m.impl("mhc_pre_bwd_c", &q38::mhc_pre_bwd_c);
}
