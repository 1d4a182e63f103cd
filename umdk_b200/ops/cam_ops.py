"""`torch.ops.umdk_cam_op_lib.*`: the four operators of the reference's torch extension with the same names,
argument order and result lists (src/cam/comm_operator/pybind/pybind.cpp:21-37; doc/en/cam/CAM API Guide.md):

    get_dispatch_layout(topk_idx, num_experts, num_ranks) -> (num_tokens_per_expert, send_token_idx_small)
    moe_dispatch_prefill(x, topk_idx, topk_weights, num_tokens_per_expert, send_token_idx_small, group_ep, rank,
                         num_ranks, use_quant) -> (recv_x, dynamic_scales, expand_idx, recv_count, recv_tokens_per_expert)
    moe_combine_prefill(x, topk_idx, topk_weights, src_idx, send_head, group_ep, rank, num_ranks) -> combined_x
    fused_deep_moe(x, expert_ids, gmm1_weight, gmm1_weight_scale, gmm2_weight, gmm2_weight_scale, expert_scales,
                   share_gmm1_weight?, ..., group_ep, ep_rank_size, ep_rank_id, moe_expert_num, quant_mode, global_bs)
                   -> [combine_x, share_output, expert_token_nums]

`group_ep` is the name under which a process group was registered with :func:`register_group` (the reference passes
the HCCL group name the same way). CUDA tensors run the sm_100a kernels, CPU tensors the gloo implementation.
Quantised dispatch uses fp8 e4m3 with a scale per 1x128 block, so `dynamic_scales` is [N, H/128] instead of the
reference's per-token int8 scale [N].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..buffer import Buffer
from . import cpu_dist
from . import reference as ref

_GROUPS: Dict[str, Buffer] = {}


def register_group(name: str, group: Optional[dist.ProcessGroup] = None, **buffer_kwargs) -> Buffer:
    """Associates `name` with a process group (None = default group) and returns the Buffer that serves it."""
    if name not in _GROUPS:
        _GROUPS[name] = Buffer(group, **buffer_kwargs)
    return _GROUPS[name]


def _buf(name: str) -> Buffer:
    if name not in _GROUPS:
        register_group(name, None)
    return _GROUPS[name]


def _load_cpp_library() -> bool:
    """Loads the C++ operator library (schemas, Meta shape functions, Autograd registration: csrc/torch_ext). Without
    it (a checkout where it was not built) the schemas are defined from Python below and there are no Meta kernels."""
    from .. import _native
    path = _native._LIB_DIR / "libumdk_cam_torch.so"
    if not path.exists():
        try:
            from .. import _build
            _build.build_all(only=["umdk_cam_torch"])
        except Exception:   # noqa: BLE001 - no compiler here: fall back to Python-side definitions
            return False
    try:
        torch.ops.load_library(str(path))
        return True
    except Exception:   # noqa: BLE001
        return False


CPP_LIBRARY_LOADED = _load_cpp_library()
if CPP_LIBRARY_LOADED:
    _lib = torch.library.Library("umdk_cam_op_lib", "FRAGMENT")
else:
    _lib = torch.library.Library("umdk_cam_op_lib", "DEF")
    _lib.define("get_dispatch_layout(Tensor topk_idx, int num_experts, int num_ranks) -> (Tensor, Tensor)")
    _lib.define("notify_dispatch(Tensor num_tokens_per_expert, Tensor num_tokens_per_rank, str group_ep, int top_k, "
                "int hidden, int max_tokens) -> (Tensor, Tensor, Tensor, Tensor)")
    _lib.define("moe_dispatch_prefill(Tensor x, Tensor topk_idx, Tensor topk_weights, Tensor num_tokens_per_expert, "
                "Tensor send_token_idx_small, str group_ep, int rank, int num_ranks, bool use_quant) -> "
                "(Tensor, Tensor, Tensor, Tensor, Tensor)")
    _lib.define("moe_combine_prefill(Tensor x, Tensor topk_idx, Tensor topk_weights, Tensor src_idx, Tensor send_head, "
                "str group_ep, int rank, int num_ranks) -> Tensor")
    _lib.define("fused_deep_moe(Tensor x, Tensor expert_ids, Tensor[] gmm1_weight, Tensor[] gmm1_weight_scale, "
                "Tensor[] gmm2_weight, Tensor[] gmm2_weight_scale, Tensor expert_scales, Tensor? share_gmm1_weight, "
                "Tensor? share_gmm1_weight_scale, Tensor? share_gmm2_weight, Tensor? share_gmm2_weight_scale, "
                "Tensor? expert_smooth_scales, Tensor? share_smooth_scales, Tensor? x_active_mask, str group_ep, "
                "int ep_rank_size, int ep_rank_id, int moe_expert_num, int quant_mode, int global_bs) -> Tensor[]")


def _get_dispatch_layout(topk_idx, num_experts, num_ranks):
    assert topk_idx.dim() == 2 and topk_idx.dtype == torch.int64, "topk_idx must be [T, K] int64"
    assert num_experts % num_ranks == 0, "num_experts must be a multiple of num_ranks"
    if topk_idx.is_cuda:
        from .ep import layout
        lay = layout(topk_idx.contiguous(), num_experts, num_ranks)
    else:
        lay = ref.ref_layout(topk_idx, num_experts, num_ranks)
    return lay.num_tokens_per_expert, lay.send_token_idx


def _notify_dispatch(num_tokens_per_expert, num_tokens_per_rank, group_ep, top_k, hidden, max_tokens):
    """Count exchange as an operator of its own -> (recv_count, recv_offset, recv_tokens_per_expert, totals). The
    reference runs it as the first half of moe_dispatch_prefill (pybind/moe_dispatch_prefill.cpp, aclnnNotifyDispatch)."""
    buf = _buf(group_ep)
    if num_tokens_per_expert.is_cuda:
        from .ep import LayoutResult
        st = buf._normal_state(num_tokens_per_expert.numel(), top_k, hidden, max_tokens)
        lay = LayoutResult(num_tokens_per_expert.to(torch.int32).contiguous(),
                           num_tokens_per_rank.to(torch.int32).contiguous(), None, None, None)
        out = st.notify(lay)
        return out.recv_count, out.recv_offset, out.recv_tokens_per_expert, out.totals
    return cpu_dist.cpu_notify(num_tokens_per_expert, num_tokens_per_rank, buf.group)


def _moe_dispatch_prefill(x, topk_idx, topk_weights, num_tokens_per_expert, send_token_idx_small, group_ep, rank,
                          num_ranks, use_quant):
    buf = _buf(group_ep)
    assert buf.group_size == num_ranks and buf.rank == rank, "group_ep does not match rank / num_ranks"
    E = num_tokens_per_expert.numel()
    T, K = topk_idx.shape
    if x.is_cuda:
        st = buf._normal_state(E, K, x.shape[1], T)
        if getattr(buf, "static_shapes", False):
            # no host synchronisation: the results keep their capacity-bound sizes (what the Meta shape function
            # reports) and recv_count says how many rows are valid
            out = st.dispatch(x.contiguous(), topk_idx.contiguous(), topk_weights.contiguous(), quant=use_quant)
            scales = out.recv_scales if use_quant else torch.empty(0, 0, dtype=torch.float32, device=x.device)
            return out.recv_x, scales, out.expand_idx.reshape(-1), out.recv_count, out.recv_tokens_per_expert
        out = st.dispatch(x.contiguous(), topk_idx.contiguous(), topk_weights.contiguous(), quant=use_quant,
                          sync_counts=True)
        n = max(out.num_recv, 0)
        scales = out.recv_scales[:n] if use_quant else torch.empty(0, dtype=torch.float32, device=x.device)
        return (out.recv_x[:n], scales, out.expand_idx[:n].reshape(-1), out.recv_count,
                out.recv_tokens_per_expert)
    res = cpu_dist.cpu_dispatch(x, topk_idx, topk_weights, E, buf.group, quant=use_quant)
    scales = res.recv_scales if use_quant else torch.empty(0, dtype=torch.float32)
    return res.recv_x, scales, res.expand_idx.reshape(-1), res.recv_count, res.recv_tokens_per_expert


def _moe_combine_prefill(x, topk_idx, topk_weights, src_idx, send_head, group_ep, rank, num_ranks):
    buf = _buf(group_ep)
    T, K = topk_idx.shape
    src = src_idx.reshape(-1, 3)
    if x.is_cuda:
        st = buf._normal_state(send_head.numel(), K, x.shape[1], T)
        return st.combine_rows(x.contiguous(), src.to(torch.int32).contiguous(), topk_idx.contiguous(),
                               topk_weights.contiguous())
    return cpu_dist.cpu_combine(x, src, topk_idx, topk_weights, T, buf.group, out_dtype=x.dtype)


# Per-expert weight LISTS (the reference's tensor-list mode, used when experts are re-placed at run time:
# op_kernel/fused_deep_moe_tiling.h:105) are not copied on every call. Tensors that already sit back to back in one
# allocation (the usual result of unbind / split of a stacked tensor) are viewed in place; anything else is stacked
# once and the result is kept for as long as the same tensors (same storage, same version) are passed again.
_STACK_CACHE: Dict[tuple, torch.Tensor] = {}
_SMOOTH_CACHE: Dict[tuple, object] = {}
_CACHE_LIMIT = 64


def _as_stacked(ws: List[torch.Tensor]) -> torch.Tensor:
    ws = list(ws)
    if len(ws) == 1 and ws[0].dim() == 3:
        return ws[0]
    first = ws[0]
    step = first.numel() * first.element_size()
    if all(w.is_contiguous() and w.shape == first.shape and w.dtype == first.dtype and
           w.untyped_storage().data_ptr() == first.untyped_storage().data_ptr() and
           w.data_ptr() == first.data_ptr() + i * step for i, w in enumerate(ws)):
        return first.as_strided((len(ws),) + tuple(first.shape), (first.numel(),) + tuple(first.stride()))
    key = tuple((w.data_ptr(), w._version, tuple(w.shape), w.dtype) for w in ws)
    hit = _STACK_CACHE.get(key)
    if hit is None:
        if len(_STACK_CACHE) >= _CACHE_LIMIT:
            _STACK_CACHE.clear()
        if first.dtype == torch.float8_e4m3fn:
            hit = torch.stack([w.view(torch.uint8) for w in ws]).contiguous().view(torch.float8_e4m3fn)
        else:
            hit = torch.stack(ws).contiguous()
        _STACK_CACHE[key] = hit
    return hit


def _fold_smooth(w, smooth: torch.Tensor):
    """Smooth-quant scales multiply the activation channel by channel before it is quantised for an expert
    (expert_smooth_scales [experts, H]). The fp8 path quantises a token once for all its experts, so the scale is
    moved to the other side of the product instead: x * s . W1^T == x . (W1 * s)^T. The rescaled, re-quantised gate /
    up weights are built once per (weights, scales) pair and reused."""
    from .ep_ll import ExpertWeights
    key = (w.w1q.data_ptr(), w.w1q._version, w.w1s.data_ptr(), smooth.data_ptr(), smooth._version, tuple(smooth.shape))
    hit = _SMOOTH_CACHE.get(key)
    if hit is None:
        if len(_SMOOTH_CACHE) >= _CACHE_LIMIT:
            _SMOOTH_CACHE.clear()
        assert smooth.shape == (w.w1q.shape[0], w.w1q.shape[2]), "smooth scales must be [local experts, hidden]"
        w1 = ref.dequant_fp8_128x128(w.w1q, w.w1s) * smooth.float().to(w.w1q.device).unsqueeze(1)
        q, s = ref.quant_fp8_128x128(w1)
        hit = ExpertWeights(q.contiguous(), s.contiguous(), w.w2q, w.w2s)
        _SMOOTH_CACHE[key] = hit
    return hit


def _fused_deep_moe(x, expert_ids, gmm1_weight, gmm1_weight_scale, gmm2_weight, gmm2_weight_scale, expert_scales,
                    share_gmm1_weight, share_gmm1_weight_scale, share_gmm2_weight, share_gmm2_weight_scale,
                    expert_smooth_scales, share_smooth_scales, x_active_mask, group_ep, ep_rank_size, ep_rank_id,
                    moe_expert_num, quant_mode, global_bs):
    from .ep_ll import ExpertWeights
    buf = _buf(group_ep)
    assert x.is_cuda, "fused_deep_moe runs on CUDA tensors"
    experts = ExpertWeights(_as_stacked(gmm1_weight), _as_stacked(gmm1_weight_scale), _as_stacked(gmm2_weight),
                            _as_stacked(gmm2_weight_scale))
    if expert_smooth_scales is not None:
        el = experts.w1q.shape[0]
        experts = _fold_smooth(experts, expert_smooth_scales[ep_rank_id * el:(ep_rank_id + 1) * el])
    shared = None
    if share_gmm1_weight is not None:
        u = lambda t: t if t.dim() == 3 else t.unsqueeze(0)
        shared = ExpertWeights(u(share_gmm1_weight), u(share_gmm1_weight_scale), u(share_gmm2_weight),
                               u(share_gmm2_weight_scale))
        if share_smooth_scales is not None:
            shared = _fold_smooth(shared, share_smooth_scales.reshape(1, -1))
    ids = expert_ids.to(torch.int64)
    if x_active_mask is not None:  # leading-true prefix mask: inactive tokens are routed nowhere
        ids = torch.where(x_active_mask.bool().unsqueeze(1), ids, torch.full_like(ids, -1))
    bs = x.shape[0]
    cap = max(bs, global_bs // max(ep_rank_size, 1)) if global_bs > 0 else bs
    out, share, cnt = buf.fused_moe(x, ids.contiguous(), expert_scales.float().contiguous(), experts, shared,
                                    num_experts=moe_expert_num, num_max_tokens_per_rank=cap)
    if share is None:
        share = torch.zeros_like(out)
    return [out, share, cnt]


for _name, _fn in (("get_dispatch_layout", _get_dispatch_layout), ("notify_dispatch", _notify_dispatch),
                   ("moe_dispatch_prefill", _moe_dispatch_prefill),
                   ("moe_combine_prefill", _moe_combine_prefill), ("fused_deep_moe", _fused_deep_moe)):
    if CPP_LIBRARY_LOADED:
        # the C++ library owns the schemas, Meta and Autograd; the kernels behind the device keys live here
        _lib.impl(_name, _fn, "CUDA")
        _lib.impl(_name, _fn, "CPU")
    else:
        _lib.impl(_name, _fn, "CompositeExplicitAutograd")
