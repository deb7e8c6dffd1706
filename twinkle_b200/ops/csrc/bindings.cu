// Python bindings of the sm_100a extension.
#include <torch/extension.h>

#include "host.h"

namespace tk {
torch::Tensor gemm(const torch::Tensor&, const torch::Tensor&, const std::string&, const c10::optional<torch::Tensor>&, bool,
                   c10::optional<torch::ScalarType>);
torch::Tensor grouped_gemm(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const std::string&, const c10::optional<torch::Tensor>&,
                           const c10::optional<torch::Tensor>&, bool, const c10::optional<torch::Tensor>&, const c10::optional<torch::Tensor>&);
torch::Tensor grouped_gemm_wgrad(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, int64_t);
std::vector<torch::Tensor> rmsnorm_fwd(const torch::Tensor&, const torch::Tensor&, double, double, const c10::optional<torch::Tensor>&);
std::vector<torch::Tensor> rmsnorm_bwd(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, double,
                                       const c10::optional<torch::Tensor>&);
std::vector<torch::Tensor> qk_norm_rope_fwd(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
                                            const torch::Tensor&, int64_t, int64_t, int64_t, double);
std::vector<torch::Tensor> qk_norm_rope_bwd(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
                                            const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
                                            const torch::Tensor&, int64_t, int64_t, int64_t);
torch::Tensor swiglu_fwd(const torch::Tensor&);
torch::Tensor swiglu_bwd(const torch::Tensor&, const torch::Tensor&);
torch::Tensor geglu_fwd(const torch::Tensor&);
torch::Tensor geglu_bwd(const torch::Tensor&, const torch::Tensor&);
void adamw_step(torch::Tensor, torch::Tensor, torch::Tensor, const torch::Tensor&, const c10::optional<torch::Tensor>&, double, double,
                double, double, double, int64_t, double);
torch::Tensor sumsq(const torch::Tensor&);
std::vector<torch::Tensor> logprob_fwd(const torch::Tensor&, const torch::Tensor&, double, bool);
torch::Tensor logprob_bwd(torch::Tensor, const torch::Tensor&, const torch::Tensor&, const c10::optional<torch::Tensor>&,
                          const torch::Tensor&, const c10::optional<torch::Tensor>&, double);
std::vector<torch::Tensor> flash_attn_fwd(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, int64_t,
                                          bool, double, const c10::optional<torch::Tensor>&);
std::vector<torch::Tensor> flash_attn_bwd(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
                                          const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, int64_t, bool, double,
                                          const c10::optional<torch::Tensor>&, int64_t);
std::tuple<torch::Tensor, py::bytes, int64_t> symm_alloc(int64_t);
int64_t symm_open(const py::bytes&);
void symm_close(int64_t);
void symm_barrier(const std::vector<int64_t>&, int64_t, int64_t, int64_t);
void peer_all_gather(torch::Tensor, const std::vector<int64_t>&, int64_t, int64_t, int64_t);
void peer_pull(const std::vector<int64_t>&, const std::vector<int64_t>&, const std::vector<int64_t>&, const std::vector<int64_t>&,
               const std::vector<int64_t>&, const std::vector<int64_t>&, int64_t);
void peer_reduce_scatter_acc(torch::Tensor, const std::vector<int64_t>&, int64_t, double, const c10::optional<torch::Tensor>&, int64_t);
void ulysses_exchange(const torch::Tensor&, const std::vector<int64_t>&, int64_t, bool, int64_t);
void peer_copy_cast(const torch::Tensor&, const std::vector<int64_t>&, int64_t);
torch::Tensor causal_conv1d_fwd(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, bool);
std::vector<torch::Tensor> gdn_recurrent_fwd(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
                                             const torch::Tensor&, const torch::Tensor&, const c10::optional<torch::Tensor>&, double, bool);
torch::Tensor paged_attn_decode(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, double);
std::vector<torch::Tensor> sample_tokens(const torch::Tensor&, double, int64_t, double, const torch::Tensor&);
std::vector<torch::Tensor> moe_router(const torch::Tensor&, int64_t, bool);
void set_gemm_pair(int64_t);
void set_gemm_staged(int64_t);
void gemm_rs(const torch::Tensor&, const torch::Tensor&, const std::string&, const std::vector<int64_t>&, int64_t);
void gemm_head_scatter(const torch::Tensor&, const torch::Tensor&, const std::vector<int64_t>&, int64_t, int64_t, int64_t, int64_t);
std::vector<torch::Tensor> gemm_ag(const std::vector<int64_t>&, int64_t, const torch::Tensor&, const std::string&, int64_t, const torch::Tensor&, int64_t, int64_t);
torch::Tensor tp_stage_reduce(const torch::Tensor&);
torch::Tensor moe_rows_gather(const torch::Tensor&, const torch::Tensor&, const c10::optional<torch::Tensor>&);
torch::Tensor moe_rows_combine(const torch::Tensor&, const torch::Tensor&, const c10::optional<torch::Tensor>&);
torch::Tensor moe_combine_wgrad(const torch::Tensor&, const torch::Tensor&, const torch::Tensor&);
torch::Tensor ep_rows_gather(const std::vector<int64_t>&, const std::vector<int64_t>&, const std::vector<int64_t>&, const torch::Tensor&, const torch::Tensor&, int64_t,
                             const torch::Tensor&, int64_t, int64_t);
torch::Tensor ep_rows_combine(const std::vector<int64_t>&, const torch::Tensor&, const torch::Tensor&, const c10::optional<torch::Tensor>&, int64_t, int64_t);
torch::Tensor ep_combine_wgrad(const torch::Tensor&, const std::vector<int64_t>&, const torch::Tensor&, const torch::Tensor&, int64_t);
}  // namespace tk

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &tk::gemm, py::arg("a"), py::arg("b"), py::arg("layout") = "nt", py::arg("out") = py::none(),
        py::arg("accumulate") = false, py::arg("out_dtype") = py::none());
  m.def("grouped_gemm", &tk::grouped_gemm, py::arg("x"), py::arg("w"), py::arg("offsets"), py::arg("layout") = "nt", py::arg("group_map") = py::none(),
        py::arg("out") = py::none(), py::arg("accumulate") = false, py::arg("x2") = py::none(), py::arg("w2") = py::none());
  m.def("grouped_gemm_wgrad", &tk::grouped_gemm_wgrad);
  m.def("rmsnorm_fwd", &tk::rmsnorm_fwd, py::arg("x"), py::arg("w"), py::arg("eps"), py::arg("offset"), py::arg("residual") = py::none());
  m.def("rmsnorm_bwd", &tk::rmsnorm_bwd, py::arg("g"), py::arg("x"), py::arg("w"), py::arg("rstd"), py::arg("offset"),
        py::arg("gadd") = py::none());
  m.def("qk_norm_rope_fwd", &tk::qk_norm_rope_fwd);
  m.def("qk_norm_rope_bwd", &tk::qk_norm_rope_bwd);
  m.def("swiglu_fwd", &tk::swiglu_fwd);
  m.def("swiglu_bwd", &tk::swiglu_bwd);
  m.def("geglu_fwd", &tk::geglu_fwd);
  m.def("geglu_bwd", &tk::geglu_bwd);
  m.def("adamw_step", &tk::adamw_step);
  m.def("sumsq", &tk::sumsq);
  m.def("logprob_fwd", &tk::logprob_fwd);
  m.def("logprob_bwd", &tk::logprob_bwd);
  m.def("flash_attn_fwd", &tk::flash_attn_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("cu"), py::arg("max_seqlen"), py::arg("causal"),
        py::arg("scale"), py::arg("cu_k") = py::none());
  m.def("flash_attn_bwd", &tk::flash_attn_bwd, py::arg("dout"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"), py::arg("cu"),
        py::arg("max_seqlen"), py::arg("causal"), py::arg("scale"), py::arg("cu_k") = py::none(), py::arg("max_seqlen_k") = 0);
  m.def("symm_alloc", &tk::symm_alloc, "cudaMalloc'ed uint8 tensor + its CUDA IPC handle");
  m.def("symm_open", &tk::symm_open);
  m.def("symm_close", &tk::symm_close);
  m.def("symm_barrier", &tk::symm_barrier, py::arg("flag_ptrs"), py::arg("rank"), py::arg("epoch"), py::arg("timeout_ms") = 3000);
  m.def("peer_all_gather", &tk::peer_all_gather);
  m.def("peer_pull", &tk::peer_pull, py::arg("src"), py::arg("dst"), py::arg("src_stride"), py::arg("dst_stride"), py::arg("chunk_bytes"),
        py::arg("rows"), py::arg("blocks_per_job"));
  m.def("peer_reduce_scatter_acc", &tk::peer_reduce_scatter_acc);
  m.def("ulysses_exchange", &tk::ulysses_exchange);
  m.def("peer_copy_cast", &tk::peer_copy_cast);
  m.def("causal_conv1d_fwd", &tk::causal_conv1d_fwd);
  m.def("gdn_recurrent_fwd", &tk::gdn_recurrent_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("g"), py::arg("beta"), py::arg("cu"),
        py::arg("init_state") = py::none(), py::arg("scale") = 1.0, py::arg("want_state") = false);
  m.def("paged_attn_decode", &tk::paged_attn_decode);
  m.def("sample_tokens", &tk::sample_tokens);
  m.def("moe_router", &tk::moe_router);
  m.def("set_gemm_pair", &tk::set_gemm_pair);
  m.def("set_gemm_staged", &tk::set_gemm_staged);
  m.def("gemm_rs", &tk::gemm_rs);
  m.def("gemm_head_scatter", &tk::gemm_head_scatter);
  m.def("gemm_ag", &tk::gemm_ag);
  m.def("tp_stage_reduce", &tk::tp_stage_reduce);
  m.def("moe_rows_gather", &tk::moe_rows_gather);
  m.def("moe_rows_combine", &tk::moe_rows_combine);
  m.def("moe_combine_wgrad", &tk::moe_combine_wgrad);
  m.def("ep_rows_gather", &tk::ep_rows_gather);
  m.def("ep_rows_combine", &tk::ep_rows_combine);
  m.def("ep_combine_wgrad", &tk::ep_combine_wgrad);
  m.def("read_and_clear_error", &tk::read_and_clear_error, "Value of the device error word (0 = healthy); clears it.");
  m.def("num_sms", &tk::num_sms);
  m.def("launch_count", &tk::launch_count, "Number of kernels launched by this extension so far.");
}
