// pybind11 surface of the sm_100a extension.  Each function is defined in its own .cu file.
#include <torch/extension.h>

namespace b200 {
void umma_gemm(std::vector<at::Tensor> a_segs, std::vector<at::Tensor> b_segs, bool a_kmajor,
               bool b_kmajor, c10::optional<at::Tensor> C, double alpha, double beta, bool sym,
               c10::optional<at::Tensor> out_hi, c10::optional<at::Tensor> out_lo, int64_t nsplit,
               c10::optional<at::Tensor> out_mid, bool split3, bool x3wide);
void set_gemm_wide(int64_t mode);
void gemm_batch_begin();
int64_t gemm_batch_end();
void gemm_batch_abort();
int64_t read_status(int64_t dev);
int64_t launch_count();
void reserve_scratch(int64_t dev, int64_t nfloats);
void cast_pad_bf16(at::Tensor src, at::Tensor hi, c10::optional<at::Tensor> lo, double scale);
void im2col_bf16(at::Tensor x, at::Tensor out, c10::optional<at::Tensor> out_lo,
                 std::vector<int64_t> kernel, std::vector<int64_t> stride,
                 std::vector<int64_t> padding, std::vector<int64_t> dilation, bool c_major);
void umma_gemm_to_ptr(std::vector<at::Tensor> a_segs, std::vector<at::Tensor> b_segs, bool a_kmajor,
                      bool b_kmajor, int64_t dst_ptr, int64_t ldc, double alpha, bool sym, int64_t atomic,
                      std::vector<int64_t> extra_ptrs, int64_t nsplit, bool mcast);
int64_t gemm_plan_new();
void gemm_plan_free(int64_t id);
void gemm_plan_add(int64_t id, std::vector<at::Tensor> a_segs, std::vector<at::Tensor> b_segs,
                   bool a_kmajor, bool b_kmajor, c10::optional<at::Tensor> C, double alpha, double beta,
                   bool sym, c10::optional<at::Tensor> out_hi, c10::optional<at::Tensor> out_lo,
                   int64_t dst_ptr, int64_t ldc, bool atomic, std::vector<int64_t> extra_ptrs,
                   int64_t nsplit, c10::optional<at::Tensor> out_mid, bool split3, bool x3wide, bool mcast);
void gemm_plan_finalize(int64_t id);
void gemm_plan_run(int64_t id);
void cast_pad_bf16_grouped(at::Tensor table, int64_t count, int64_t max_elems);
void cast_split3(at::Tensor src, at::Tensor hi, at::Tensor mid, at::Tensor lo);
void transpose_cast(at::Tensor src, at::Tensor dst);
void bn_unitwise_stats(at::Tensor y, at::Tensor g, at::Tensor weight, at::Tensor bias, at::Tensor stats,
                       double alpha, double beta);
std::vector<at::Tensor> bn_forward_train(at::Tensor x, at::Tensor weight, at::Tensor bias,
                                         c10::optional<at::Tensor> running_mean,
                                         c10::optional<at::Tensor> running_var,
                                         c10::optional<at::Tensor> num_batches_tracked, double momentum,
                                         double eps, c10::optional<at::Tensor> residual, bool relu);
std::vector<at::Tensor> bn_backward_train(at::Tensor x, at::Tensor dy, at::Tensor weight, at::Tensor mean,
                                          at::Tensor invstd, c10::optional<at::Tensor> y, bool want_dres,
                                          c10::optional<at::Tensor> bias_for_mask);
void bn_unitwise_stats_xhat(at::Tensor x, at::Tensor dy, c10::optional<at::Tensor> y, at::Tensor mean,
                            at::Tensor invstd, at::Tensor stats, double alpha, double beta);
bool ln_supported_size(int64_t d);
std::vector<at::Tensor> ln_forward(at::Tensor x, at::Tensor weight, at::Tensor bias, double eps);
std::vector<at::Tensor> ln_backward(at::Tensor x, at::Tensor dy, at::Tensor weight, at::Tensor mean,
                                    at::Tensor rstd);
void symm_barrier(at::Tensor peers, int64_t rank, int64_t world, int64_t slot, int64_t wait_ms);
void symm_reduce_segments(at::Tensor peers, int64_t rank, int64_t world, at::Tensor segs, double scale,
                          int64_t mc_ptr);
void symm_bcast_segments(at::Tensor peers, int64_t rank, int64_t world, at::Tensor segs, int64_t mc_ptr);
void symm_bucket_reduce(at::Tensor peers, int64_t rank, int64_t world, int64_t slot, at::Tensor segs, double scale,
                        int64_t mc_ptr, int64_t wait_ms, int64_t blocks);
void symm_scale_segments(at::Tensor local, at::Tensor segs, double beta);
void symm_mirror_lower(at::Tensor local, at::Tensor mats, int64_t n_max);
void symm_pull_slots(at::Tensor local, at::Tensor peers, at::Tensor table, int64_t world, int64_t n_max, double beta);
void symm_reduce_slots(at::Tensor local, at::Tensor table, int64_t world, int64_t slot_stride, int64_t n_max,
                       double beta);
void chol_inverse(std::vector<at::Tensor> mats, std::vector<at::Tensor> outs, at::Tensor damping);
void chol_inverse_tc(std::vector<at::Tensor> mats, std::vector<at::Tensor> outs, at::Tensor damping);
void chol_inverse_tc_clear_cache();
std::vector<at::Tensor> jacobi_eigh(at::Tensor mats, bool want_vectors);
void ln_unitwise_stats(at::Tensor y, at::Tensor g, at::Tensor weight, at::Tensor bias, at::Tensor stats, double alpha,
                       double beta);
void unitwise_inverse_mt(std::vector<std::vector<int64_t>> rows, double damping);
void unitwise_apply_mt(std::vector<std::vector<int64_t>> rows, double grad_scale);
void bias_precondition_mt(std::vector<std::vector<int64_t>> rows, double grad_scale);
at::Tensor batched_mv(at::Tensor a, at::Tensor x);
void embedding_diag_stats(at::Tensor idx, at::Tensor g, at::Tensor out, int64_t padding_idx, double scale);
void embedding_counts(at::Tensor idx, at::Tensor counts);
void bfgs_powell_damping(at::Tensor H, at::Tensor s, at::Tensor y, double mu1, double mu2);
void bfgs_inv_update(at::Tensor H, at::Tensor s, at::Tensor y);
void umma_syrk_conv(at::Tensor x, c10::optional<at::Tensor> C, int64_t kh, int64_t kw, int64_t ph, int64_t pw,
                    double alpha, double beta, int64_t nsplit_req, int64_t dst_ptr, int64_t ldc, int64_t mode);
void gram_hadamard(std::vector<at::Tensor> a1, std::vector<at::Tensor> a2, std::vector<at::Tensor> g1,
                   std::vector<at::Tensor> g2, at::Tensor kernel, double alpha, double one);
void diag_linear_stats(at::Tensor a, at::Tensor g, at::Tensor out, c10::optional<at::Tensor> out_bias, double alpha,
                       double beta);
}  // namespace b200

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("umma_gemm", &b200::umma_gemm, "tcgen05 TN GEMM / SYRK", py::arg("a_segs"),
        py::arg("b_segs"), py::arg("a_kmajor"), py::arg("b_kmajor"), py::arg("C"),
        py::arg("alpha"), py::arg("beta"), py::arg("sym"), py::arg("out_hi"), py::arg("out_lo"),
        py::arg("nsplit"), py::arg("out_mid") = py::none(), py::arg("split3") = false, py::arg("x3wide") = false);
  m.def("set_gemm_wide", &b200::set_gemm_wide);
  m.def("gemm_batch_begin", &b200::gemm_batch_begin);
  m.def("gemm_batch_end", &b200::gemm_batch_end);
  m.def("gemm_batch_abort", &b200::gemm_batch_abort);
  m.def("read_status", &b200::read_status);
  m.def("launch_count", &b200::launch_count);
  m.def("reserve_scratch", &b200::reserve_scratch);
  m.def("cast_pad_bf16", &b200::cast_pad_bf16);
  m.def("im2col_bf16", &b200::im2col_bf16);
  m.def("umma_gemm_to_ptr", &b200::umma_gemm_to_ptr, py::arg("a_segs"), py::arg("b_segs"), py::arg("a_kmajor"),
        py::arg("b_kmajor"), py::arg("dst_ptr"), py::arg("ldc"), py::arg("alpha"), py::arg("sym"), py::arg("atomic"),
        py::arg("extra_ptrs"), py::arg("nsplit"), py::arg("mcast") = false);
  m.def("gemm_plan_new", &b200::gemm_plan_new);
  m.def("gemm_plan_free", &b200::gemm_plan_free);
  m.def("gemm_plan_add", &b200::gemm_plan_add, py::arg("plan"), py::arg("a_segs"), py::arg("b_segs"),
        py::arg("a_kmajor"), py::arg("b_kmajor"), py::arg("C"), py::arg("alpha"), py::arg("beta"), py::arg("sym"),
        py::arg("out_hi"), py::arg("out_lo"), py::arg("dst_ptr"), py::arg("ldc"), py::arg("atomic"),
        py::arg("extra_ptrs"), py::arg("nsplit"), py::arg("out_mid") = py::none(), py::arg("split3") = false, py::arg("x3wide") = false, py::arg("mcast") = false);
  m.def("gemm_plan_finalize", &b200::gemm_plan_finalize);
  m.def("gemm_plan_run", &b200::gemm_plan_run);
  m.def("cast_pad_bf16_grouped", &b200::cast_pad_bf16_grouped, py::arg("table"), py::arg("count"), py::arg("max_elems") = 0);
  m.def("cast_split3", &b200::cast_split3);
  m.def("transpose_cast", &b200::transpose_cast);
  m.def("bn_unitwise_stats", &b200::bn_unitwise_stats);
  m.def("bn_forward_train", &b200::bn_forward_train);
  m.def("bn_backward_train", &b200::bn_backward_train);
  m.def("bn_unitwise_stats_xhat", &b200::bn_unitwise_stats_xhat);
  m.def("ln_supported_size", &b200::ln_supported_size);
  m.def("ln_forward", &b200::ln_forward);
  m.def("ln_backward", &b200::ln_backward);
  m.def("symm_barrier", &b200::symm_barrier);
  m.def("symm_reduce_segments", &b200::symm_reduce_segments, py::arg("peers"), py::arg("rank"), py::arg("world"),
        py::arg("segs"), py::arg("scale"), py::arg("mc_ptr") = 0);
  m.def("symm_bcast_segments", &b200::symm_bcast_segments, py::arg("peers"), py::arg("rank"), py::arg("world"),
        py::arg("segs"), py::arg("mc_ptr") = 0);
  m.def("symm_bucket_reduce", &b200::symm_bucket_reduce);
  m.def("symm_scale_segments", &b200::symm_scale_segments);
  m.def("symm_mirror_lower", &b200::symm_mirror_lower);
  m.def("symm_reduce_slots", &b200::symm_reduce_slots);
  m.def("symm_pull_slots", &b200::symm_pull_slots);
  m.def("chol_inverse", &b200::chol_inverse, "grouped damped SPD inverse (fp32, CUDA cores)");
  m.def("chol_inverse_tc", &b200::chol_inverse_tc, "grouped damped SPD inverse (fp32-accurate, tensor cores)");
  m.def("chol_inverse_tc_clear_cache", &b200::chol_inverse_tc_clear_cache);
  m.def("jacobi_eigh", &b200::jacobi_eigh, "batched symmetric eigendecomposition, n <= 128 (parallel cyclic Jacobi)");
  m.def("ln_unitwise_stats", &b200::ln_unitwise_stats);
  m.def("unitwise_inverse_mt", &b200::unitwise_inverse_mt);
  m.def("unitwise_apply_mt", &b200::unitwise_apply_mt);
  m.def("bias_precondition_mt", &b200::bias_precondition_mt);
  m.def("diag_linear_stats", &b200::diag_linear_stats);
  m.def("batched_mv", &b200::batched_mv);
  m.def("embedding_diag_stats", &b200::embedding_diag_stats, "out[idx[t], :] += scale * g[t, :]^2 (reductions, no sort)");
  m.def("embedding_counts", &b200::embedding_counts, "counts[example, idx] += 1");
  m.def("bfgs_powell_damping", &b200::bfgs_powell_damping, "Powell damping + LM shift of a BFGS pair, in place");
  m.def("bfgs_inv_update", &b200::bfgs_inv_update, "symmetrise H and apply the rank-2 BFGS update of the inverse, in place");
  m.def("umma_syrk_conv", &b200::umma_syrk_conv,
        "alpha * M^T M (+ beta * C) for the patch matrix M of a stride-1 convolution input, gathered by 4-d TMA boxes",
        py::arg("x"), py::arg("C"), py::arg("kh"), py::arg("kw"), py::arg("ph"), py::arg("pw"), py::arg("alpha"),
        py::arg("beta"), py::arg("nsplit"), py::arg("dst_ptr") = 0, py::arg("ldc") = 0, py::arg("mode") = 0);
  m.def("gram_hadamard", &b200::gram_hadamard,
        "kernel += alpha * (A1 A2^T + one) o (G1 G2^T), both Gram tiles in TMEM, multiplied in the epilogue");
}
