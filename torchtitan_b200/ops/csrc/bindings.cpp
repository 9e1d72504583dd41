// Operator registration: everything is exposed under torch.ops.tb200.
#include <ATen/ATen.h>
#include <torch/library.h>

namespace tb200 {
std::tuple<at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& w, double eps);
std::tuple<at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x,
                                               const c10::optional<at::Tensor>& w, const at::Tensor& rstd);
void rope_(at::Tensor x, const at::Tensor& table, const at::Tensor& positions, bool interleaved, bool inverse);
at::Tensor swiglu_fwd(const at::Tensor& gu);
at::Tensor swiglu_bwd(const at::Tensor& gu, const at::Tensor& dout);
std::tuple<at::Tensor, at::Tensor, at::Tensor> mla_assemble_fwd(const at::Tensor& q, const at::Tensor& kv, const at::Tensor& k_pe,
                                                                const at::Tensor& table, const at::Tensor& positions, int64_t dn,
                                                                int64_t dr, int64_t dv);
std::tuple<at::Tensor, at::Tensor, at::Tensor> mla_assemble_bwd(const at::Tensor& dqf, const at::Tensor& dkf, const at::Tensor& dv_,
                                                                const at::Tensor& table, const at::Tensor& positions, int64_t dn,
                                                                int64_t dr, int64_t dv);
at::Tensor conv_silu_fwd(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& pos);
std::tuple<at::Tensor, at::Tensor> conv_silu_bwd(const at::Tensor& x, const at::Tensor& w,
                                                 const c10::optional<at::Tensor>& pos, const at::Tensor& dy);
int64_t status(bool clear);
at::Tensor cross_entropy_(at::Tensor logits, const at::Tensor& labels, const at::Tensor& scale);
void adamw_(at::Tensor master, const at::Tensor& grad, at::Tensor exp_avg, at::Tensor exp_avg_sq,
            const c10::optional<at::Tensor>& lowp, const at::Tensor& grad_scale, double lr, double beta1,
            double beta2, double eps, double weight_decay, double bc1, double bc2);
void sumsq_(const at::Tensor& x, at::Tensor acc);
void gemm_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor c, int64_t mode, bool accumulate);
void gemm_grouped_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor c, const at::Tensor& offs, int64_t mode,
                       int64_t align, bool accumulate);
void gemm_allgather_bf16(const at::Tensor& a_gather, const at::Tensor& b, at::Tensor c, at::IntArrayRef peer_ptrs,
                         int64_t rank, at::Tensor flags, const at::Tensor& epoch, int64_t mode);
void gemm_scatter_bf16(const at::Tensor& a, const at::Tensor& b, at::IntArrayRef staging_ptrs, int64_t rank, int64_t mode);
at::Tensor sum_slots(const at::Tensor& staging);
int64_t gemm_status(bool clear);
void gemm_set_variant(int64_t v);
void gemm_set_mn3d(int64_t v);
void gemm_set_debug(int64_t v);
std::tuple<at::Tensor, at::Tensor> flash_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale,
                                             bool causal, int64_t causal_offset,
                                             const c10::optional<at::Tensor>& kv_first, int64_t window,
                                             const c10::optional<at::Tensor>& sinks);
void flash_set_fwd_variant(int64_t v);
void attn_merge_(at::Tensor acc_o, at::Tensor acc_lse, const at::Tensor& o, const at::Tensor& lse);
std::tuple<at::Tensor, at::Tensor, at::Tensor> flash_bwd(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k,
                                                         const at::Tensor& v, const at::Tensor& o, const at::Tensor& lse,
                                                         double scale, bool causal, int64_t causal_offset,
                                                         const c10::optional<at::Tensor>& kv_first,
                                                         const c10::optional<at::Tensor>& dq_out,
                                                         const c10::optional<at::Tensor>& dk_out,
                                                         const c10::optional<at::Tensor>& dv_out, int64_t window);
int64_t flash_status(bool clear);
void flash_set_debug(int64_t v);
void symm_barrier(at::IntArrayRef flag_ptrs, int64_t my_rank, at::Tensor epoch, at::Tensor status, int64_t max_cycles,
                  const c10::optional<at::Tensor>& bump);
void all_gather_pull(at::IntArrayRef src_ptrs, int64_t my_rank, int64_t nbytes, at::Tensor out);
void reduce_scatter_pull(at::IntArrayRef grad_ptrs, int64_t my_rank, int64_t offset, at::Tensor out, bool grad_is_bf16,
                         bool accumulate);
void adamw_allgather_(at::Tensor master, const at::Tensor& grad, at::Tensor exp_avg, at::Tensor exp_avg_sq,
                      at::IntArrayRef param_ptrs, int64_t my_rank, int64_t offset, bool param_is_bf16,
                      int64_t multicast_ptr, const at::Tensor& grad_scale, double lr, double beta1, double beta2, double eps,
                      double weight_decay, double bc1, double bc2);
std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_router_fwd(const at::Tensor& logits, const c10::optional<at::Tensor>& bias,
                                                              int64_t top_k, bool sigmoid, bool route_norm,
                                                              double route_scale);
at::Tensor moe_router_bwd(const at::Tensor& logits, const at::Tensor& sel, const at::Tensor& dtop, bool sigmoid,
                          bool route_norm, double route_scale);
at::Tensor moe_permute_rows(const at::Tensor& x, const at::Tensor& dest, int64_t rows);
at::Tensor moe_combine_rows(const at::Tensor& y, const at::Tensor& dest, const c10::optional<at::Tensor>& wts);
std::tuple<at::Tensor, at::Tensor> moe_combine_bwd(const at::Tensor& dout, const at::Tensor& y, const at::Tensor& dest,
                                                   const at::Tensor& wts);
void ep_scatter_rows(const at::Tensor& x, const at::Tensor& dest_rank, const at::Tensor& dest_row,
                     const c10::optional<at::Tensor>& wts, at::IntArrayRef peer_ptrs);
std::tuple<at::Tensor, at::Tensor> ep_gather_rows(at::IntArrayRef peer_ptrs, const at::Tensor& dest_rank,
                                                  const at::Tensor& dest_row, const c10::optional<at::Tensor>& wts,
                                                  int64_t D, bool keep_rows, const at::Tensor& like);
void moe_zero_pad_rows(at::Tensor buf, const at::Tensor& offs, const at::Tensor& counts);
void ep_publish_counts(const at::Tensor& counts, at::IntArrayRef table_ptrs, int64_t my_rank);
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> ep_layout(const at::Tensor& selected, const at::Tensor& table,
                                                                     int64_t my_rank, int64_t cap, int64_t align,
                                                                     at::Tensor status);
at::Tensor moe_slot_dot(const at::Tensor& dout, const at::Tensor& rows, int64_t K);
std::tuple<at::Tensor, at::Tensor> mxfp8_quantize(const at::Tensor& x, int64_t axis);
at::Tensor mxfp8_fake_quant(const at::Tensor& x, int64_t axis);
std::tuple<at::Tensor, at::Tensor> mxfp8_quantize_tiled(const at::Tensor& x);
at::Tensor gemm_mxfp8(const at::Tensor& a, const at::Tensor& sfa, const at::Tensor& b, const at::Tensor& sfb);
void gemm_mx_set_variant(int64_t v);
at::Tensor gemm_mxfp8_grouped(const at::Tensor& a, const at::Tensor& sfa, const at::Tensor& b, const at::Tensor& sfb,
                              const at::Tensor& offs, int64_t mode);
void gemm_mx_set_debug(int64_t v);
std::tuple<at::Tensor, at::Tensor> mxfp8_quantize_tiled_t(const at::Tensor& x);
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> mxfp8_quantize_tiled_both(const at::Tensor& x);
std::tuple<at::Tensor, at::Tensor> float8_pow2_quantize_tiled(const at::Tensor& x, const at::Tensor& exps);
std::tuple<at::Tensor, at::Tensor> float8_pow2_quantize_tiled_t(const at::Tensor& x, const at::Tensor& exps);
at::Tensor mxfp8_dequantize(const at::Tensor& data, const at::Tensor& scales, int64_t axis);
std::tuple<at::Tensor, at::Tensor> float8_rowwise_quantize(const at::Tensor& x);
at::Tensor float8_rowwise_fake_quant(const at::Tensor& x);
}  // namespace tb200

TORCH_LIBRARY(tb200, m) {
  m.def("rmsnorm_fwd(Tensor x, Tensor? w, float eps) -> (Tensor, Tensor)", &tb200::rmsnorm_fwd);
  m.def("rmsnorm_bwd(Tensor dy, Tensor x, Tensor? w, Tensor rstd) -> (Tensor, Tensor)", &tb200::rmsnorm_bwd);
  m.def("rope_(Tensor(a!) x, Tensor table, Tensor positions, bool interleaved, bool inverse) -> ()", &tb200::rope_);
  m.def("swiglu_fwd(Tensor gu) -> Tensor", &tb200::swiglu_fwd);
  m.def("swiglu_bwd(Tensor gu, Tensor dout) -> Tensor", &tb200::swiglu_bwd);
  m.def("mla_assemble_fwd(Tensor q, Tensor kv, Tensor k_pe, Tensor table, Tensor positions, int dn, int dr, int dv) -> (Tensor, Tensor, Tensor)",
        &tb200::mla_assemble_fwd);
  m.def("mla_assemble_bwd(Tensor dqf, Tensor dkf, Tensor dv, Tensor table, Tensor positions, int dn, int dr, int dv) -> (Tensor, Tensor, Tensor)",
        &tb200::mla_assemble_bwd);
  m.def("conv_silu_fwd(Tensor x, Tensor w, Tensor? pos) -> Tensor", &tb200::conv_silu_fwd);
  m.def("conv_silu_bwd(Tensor x, Tensor w, Tensor? pos, Tensor dy) -> (Tensor, Tensor)", &tb200::conv_silu_bwd);
  m.def("status(bool clear) -> int", &tb200::status);
  m.def("cross_entropy_(Tensor(a!) logits, Tensor labels, Tensor scale) -> Tensor", &tb200::cross_entropy_);
  m.def("adamw_(Tensor(a!) master, Tensor grad, Tensor(b!) exp_avg, Tensor(c!) exp_avg_sq, Tensor(d!)? lowp, "
        "Tensor grad_scale, float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2) -> ()",
        &tb200::adamw_);
  m.def("sumsq_(Tensor x, Tensor(a!) acc) -> ()", &tb200::sumsq_);
  m.def("gemm_bf16(Tensor a, Tensor b, Tensor(a!) c, int mode, bool accumulate) -> ()", &tb200::gemm_bf16);
  m.def("gemm_grouped_bf16(Tensor a, Tensor b, Tensor(a!) c, Tensor offs, int mode, int align, bool accumulate) -> ()",
        &tb200::gemm_grouped_bf16);
  m.def("gemm_allgather_bf16(Tensor(a!) a_gather, Tensor b, Tensor(b!) c, int[] peer_ptrs, int rank, Tensor(c!) flags, "
        "Tensor epoch, int mode) -> ()", &tb200::gemm_allgather_bf16);
  m.def("gemm_scatter_bf16(Tensor a, Tensor b, int[] staging_ptrs, int rank, int mode) -> ()", &tb200::gemm_scatter_bf16);
  m.def("sum_slots(Tensor staging) -> Tensor", &tb200::sum_slots);
  m.def("gemm_status(bool clear) -> int", &tb200::gemm_status);
  m.def("gemm_set_variant(int v) -> ()", &tb200::gemm_set_variant);
  m.def("gemm_set_mn3d(int v) -> ()", &tb200::gemm_set_mn3d);
  m.def("gemm_set_debug(int v) -> ()", &tb200::gemm_set_debug);
  m.def("flash_fwd(Tensor q, Tensor k, Tensor v, float scale, bool causal, int causal_offset, Tensor? kv_first, "
        "int window=0, Tensor? sinks=None) -> (Tensor, Tensor)", &tb200::flash_fwd);
  m.def("flash_set_fwd_variant(int v) -> ()", &tb200::flash_set_fwd_variant);
  m.def("attn_merge_(Tensor(a!) acc_o, Tensor(b!) acc_lse, Tensor o, Tensor lse) -> ()", &tb200::attn_merge_);
  m.def("flash_bwd(Tensor d_o, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, float scale, bool causal, "
        "int causal_offset, Tensor? kv_first, Tensor(a!)? dq_out, Tensor(b!)? dk_out, Tensor(c!)? dv_out, "
        "int window=0) -> (Tensor, Tensor, Tensor)", &tb200::flash_bwd);
  m.def("flash_status(bool clear) -> int", &tb200::flash_status);
  m.def("flash_set_debug(int v) -> ()", &tb200::flash_set_debug);
  m.def("ep_scatter_rows(Tensor x, Tensor dest_rank, Tensor dest_row, Tensor? wts, int[] peer_ptrs) -> ()", &tb200::ep_scatter_rows);
  m.def("ep_gather_rows(int[] peer_ptrs, Tensor dest_rank, Tensor dest_row, Tensor? wts, int D, bool keep_rows, Tensor like) -> "
        "(Tensor, Tensor)", &tb200::ep_gather_rows);
  m.def("moe_zero_pad_rows(Tensor(a!) buf, Tensor offs, Tensor counts) -> ()", &tb200::moe_zero_pad_rows);
  m.def("ep_publish_counts(Tensor counts, int[] table_ptrs, int my_rank) -> ()", &tb200::ep_publish_counts);
  m.def("ep_layout(Tensor selected, Tensor table, int my_rank, int cap, int align, Tensor(a!) status) -> "
        "(Tensor, Tensor, Tensor, Tensor)", &tb200::ep_layout);
  m.def("moe_slot_dot(Tensor dout, Tensor rows, int K) -> Tensor", &tb200::moe_slot_dot);
  m.def("mxfp8_quantize(Tensor x, int axis) -> (Tensor, Tensor)", &tb200::mxfp8_quantize);
  m.def("mxfp8_fake_quant(Tensor x, int axis) -> Tensor", &tb200::mxfp8_fake_quant);
  m.def("mxfp8_quantize_tiled(Tensor x) -> (Tensor, Tensor)", &tb200::mxfp8_quantize_tiled);
  m.def("gemm_mxfp8(Tensor a, Tensor sfa, Tensor b, Tensor sfb) -> Tensor", &tb200::gemm_mxfp8);
  m.def("gemm_mx_set_variant(int v) -> ()", &tb200::gemm_mx_set_variant);
  m.def("gemm_mxfp8_grouped(Tensor a, Tensor sfa, Tensor b, Tensor sfb, Tensor offs, int mode) -> Tensor", &tb200::gemm_mxfp8_grouped);
  m.def("gemm_mx_set_debug(int v) -> ()", &tb200::gemm_mx_set_debug);
  m.def("mxfp8_quantize_tiled_t(Tensor x) -> (Tensor, Tensor)", &tb200::mxfp8_quantize_tiled_t);
  m.def("mxfp8_quantize_tiled_both(Tensor x) -> (Tensor, Tensor, Tensor, Tensor)", &tb200::mxfp8_quantize_tiled_both);
  m.def("float8_pow2_quantize_tiled(Tensor x, Tensor exps) -> (Tensor, Tensor)", &tb200::float8_pow2_quantize_tiled);
  m.def("float8_pow2_quantize_tiled_t(Tensor x, Tensor exps) -> (Tensor, Tensor)", &tb200::float8_pow2_quantize_tiled_t);
  m.def("mxfp8_dequantize(Tensor data, Tensor scales, int axis) -> Tensor", &tb200::mxfp8_dequantize);
  m.def("float8_rowwise_quantize(Tensor x) -> (Tensor, Tensor)", &tb200::float8_rowwise_quantize);
  m.def("float8_rowwise_fake_quant(Tensor x) -> Tensor", &tb200::float8_rowwise_fake_quant);
  m.def("moe_router_fwd(Tensor logits, Tensor? bias, int top_k, bool sigmoid, bool route_norm, float route_scale) -> "
        "(Tensor, Tensor, Tensor)", &tb200::moe_router_fwd);
  m.def("moe_router_bwd(Tensor logits, Tensor sel, Tensor dtop, bool sigmoid, bool route_norm, float route_scale) -> Tensor",
        &tb200::moe_router_bwd);
  m.def("moe_permute_rows(Tensor x, Tensor dest, int rows) -> Tensor", &tb200::moe_permute_rows);
  m.def("moe_combine_rows(Tensor y, Tensor dest, Tensor? wts) -> Tensor", &tb200::moe_combine_rows);
  m.def("moe_combine_bwd(Tensor dout, Tensor y, Tensor dest, Tensor wts) -> (Tensor, Tensor)", &tb200::moe_combine_bwd);
  m.def("symm_barrier(int[] flag_ptrs, int my_rank, Tensor(a!) epoch, Tensor(b!) status, int max_cycles, Tensor(c!)? bump=None) -> ()",
        &tb200::symm_barrier);
  m.def("all_gather_pull(int[] src_ptrs, int my_rank, int nbytes, Tensor(a!) out) -> ()", &tb200::all_gather_pull);
  m.def("reduce_scatter_pull(int[] grad_ptrs, int my_rank, int offset, Tensor(a!) out, bool grad_is_bf16, "
        "bool accumulate) -> ()", &tb200::reduce_scatter_pull);
  m.def("adamw_allgather_(Tensor(a!) master, Tensor grad, Tensor(b!) exp_avg, Tensor(c!) exp_avg_sq, int[] param_ptrs, "
        "int my_rank, int offset, bool param_is_bf16, int multicast_ptr, Tensor grad_scale, float lr, float beta1, float beta2, float eps, "
        "float weight_decay, float bc1, float bc2) -> ()", &tb200::adamw_allgather_);
}
