// Operator library `umdk_cam_op_lib` registered from C++: schemas, shape functions for the Meta key (so that fake-tensor
// tracing, torch.export and torch.compile see the operators without running a kernel), and an Autograd registration
// that marks the operators as not differentiable. The kernels behind the CUDA and CPU keys are registered by the
// Python package on the same library (umdk_b200/ops/cam_ops.py): they need the process-group and symmetric-heap
// state that lives there. The reference project registers its operators the same way for its device key, its Autograd
// key and Meta (src/cam/comm_operator/pybind/pybind.cpp:21-37, fused_deep_moe.cpp:91-124, 246-259).
#include <torch/library.h>
#include <ATen/ATen.h>
#include <torch/csrc/autograd/autograd_not_implemented_fallback.h>

#include <tuple>
#include <vector>

namespace {

using at::Tensor;

std::tuple<Tensor, Tensor> layout_meta(const Tensor& topk_idx, int64_t num_experts, int64_t num_ranks) {
  TORCH_CHECK(topk_idx.dim() == 2, "topk_idx must be [T, K]");
  TORCH_CHECK(num_ranks > 0 && num_experts % num_ranks == 0, "num_experts must be a multiple of num_ranks");
  auto i32 = topk_idx.options().dtype(at::kInt);
  return {at::empty({num_experts}, i32), at::empty_symint(topk_idx.sym_sizes(), i32)};
}

std::tuple<Tensor, Tensor, Tensor, Tensor> notify_meta(const Tensor& num_tokens_per_expert,
                                                       const Tensor& num_tokens_per_rank, c10::string_view,
                                                       int64_t, int64_t, int64_t) {
  const int64_t E = num_tokens_per_expert.numel();
  const int64_t R = num_tokens_per_rank.numel();
  TORCH_CHECK(R > 0 && E % R == 0, "num_tokens_per_expert / num_tokens_per_rank sizes do not match");
  auto i32 = num_tokens_per_expert.options().dtype(at::kInt);
  return {at::empty({E}, i32), at::empty({E}, i32), at::empty({E / R}, i32.dtype(at::kLong)), at::empty({4}, i32)};
}

// Dispatch returns as many rows as other ranks send, which only the run knows: the Meta function reports the
// capacity bound R * T * min(K, E / R); callers that trace with fake tensors slice by `recv_count[-1]` afterwards.
// (The Python package overrides this with a data-dependent size when torch can express one.)
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> dispatch_meta(const Tensor& x, const Tensor& topk_idx,
                                                                 const Tensor&, const Tensor& num_tokens_per_expert,
                                                                 const Tensor&, c10::string_view, int64_t,
                                                                 int64_t num_ranks, bool use_quant) {
  TORCH_CHECK(x.dim() == 2 && topk_idx.dim() == 2, "x must be [T, H] and topk_idx [T, K]");
  const int64_t T = x.size(0), H = x.size(1), K = topk_idx.size(1), E = num_tokens_per_expert.numel();
  const int64_t el = E / std::max<int64_t>(num_ranks, 1);
  const int64_t n = num_ranks * T * std::min(K, el);
  auto i32 = topk_idx.options().dtype(at::kInt);
  Tensor recv = use_quant ? at::empty({n, H}, x.options().dtype(at::kFloat8_e4m3fn)) : at::empty({n, H}, x.options());
  Tensor scales = at::empty({use_quant ? n : 0, use_quant ? H / 128 : 0}, x.options().dtype(at::kFloat));
  return {recv, scales, at::empty({n * 3}, i32), at::empty({E}, i32), at::empty({el}, i32.dtype(at::kLong))};
}

Tensor combine_meta(const Tensor& x, const Tensor& topk_idx, const Tensor&, const Tensor&, const Tensor&,
                    c10::string_view, int64_t, int64_t) {
  TORCH_CHECK(x.dim() == 2 && topk_idx.dim() == 2, "x must be [N, H] and topk_idx [T, K]");
  return at::empty_symint({topk_idx.sym_size(0), x.sym_size(1)}, x.options());
}

std::vector<Tensor> fused_deep_moe_meta(const Tensor& x, const Tensor& expert_ids, at::TensorList, at::TensorList,
                                        at::TensorList, at::TensorList, const Tensor&,
                                        const c10::optional<Tensor>&, const c10::optional<Tensor>&,
                                        const c10::optional<Tensor>&, const c10::optional<Tensor>&,
                                        const c10::optional<Tensor>&, const c10::optional<Tensor>&,
                                        const c10::optional<Tensor>&, c10::string_view, int64_t ep_rank_size, int64_t,
                                        int64_t moe_expert_num, int64_t, int64_t) {
  TORCH_CHECK(x.dim() == 2 && expert_ids.dim() == 2, "x must be [T, H] and expert_ids [T, K]");
  TORCH_CHECK(ep_rank_size > 0 && moe_expert_num % ep_rank_size == 0, "moe_expert_num must divide by ep_rank_size");
  Tensor out = at::empty_symint(x.sym_sizes(), x.options());
  Tensor share = at::empty_symint(x.sym_sizes(), x.options());
  Tensor cnt = at::empty({moe_expert_num / ep_rank_size}, expert_ids.options().dtype(at::kLong));
  return {out, share, cnt};
}

}  // namespace

TORCH_LIBRARY(umdk_cam_op_lib, m) {
  m.def("get_dispatch_layout(Tensor topk_idx, int num_experts, int num_ranks) -> (Tensor, Tensor)");
  m.def("notify_dispatch(Tensor num_tokens_per_expert, Tensor num_tokens_per_rank, str group_ep, int top_k, "
        "int hidden, int max_tokens) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("moe_dispatch_prefill(Tensor x, Tensor topk_idx, Tensor topk_weights, Tensor num_tokens_per_expert, "
        "Tensor send_token_idx_small, str group_ep, int rank, int num_ranks, bool use_quant) -> "
        "(Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("moe_combine_prefill(Tensor x, Tensor topk_idx, Tensor topk_weights, Tensor src_idx, Tensor send_head, "
        "str group_ep, int rank, int num_ranks) -> Tensor");
  m.def("fused_deep_moe(Tensor x, Tensor expert_ids, Tensor[] gmm1_weight, Tensor[] gmm1_weight_scale, "
        "Tensor[] gmm2_weight, Tensor[] gmm2_weight_scale, Tensor expert_scales, Tensor? share_gmm1_weight, "
        "Tensor? share_gmm1_weight_scale, Tensor? share_gmm2_weight, Tensor? share_gmm2_weight_scale, "
        "Tensor? expert_smooth_scales, Tensor? share_smooth_scales, Tensor? x_active_mask, str group_ep, "
        "int ep_rank_size, int ep_rank_id, int moe_expert_num, int quant_mode, int global_bs) -> Tensor[]");
}

TORCH_LIBRARY_IMPL(umdk_cam_op_lib, Meta, m) {
  m.impl("get_dispatch_layout", &layout_meta);
  m.impl("notify_dispatch", &notify_meta);
  m.impl("moe_dispatch_prefill", &dispatch_meta);
  m.impl("moe_combine_prefill", &combine_meta);
  m.impl("fused_deep_moe", &fused_deep_moe_meta);
}

// Inference operators: gradients are not defined; asking for one raises instead of silently returning zeros.
TORCH_LIBRARY_IMPL(umdk_cam_op_lib, Autograd, m) {
  m.impl("get_dispatch_layout", torch::autograd::autogradNotImplementedFallback());
  m.impl("notify_dispatch", torch::autograd::autogradNotImplementedFallback());
  m.impl("moe_dispatch_prefill", torch::autograd::autogradNotImplementedFallback());
  m.impl("moe_combine_prefill", torch::autograd::autogradNotImplementedFallback());
  m.impl("fused_deep_moe", torch::autograd::autogradNotImplementedFallback());
}

extern "C" __attribute__((visibility("default"))) int umdk_cam_torch_ops_abi() { return 1; }
