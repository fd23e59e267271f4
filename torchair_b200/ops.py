"""torch.ops.npu.* operators of the W8A8 MoE path, registered with torch.library and backed by the C ABI.

Schemas keep the names, argument order, keyword names and defaults that the reference's converters bind to
(python/torchair/_ge_concrete_graph/ge_converter/custom/{moe_init_routing, npu_dynamic_quant, npu_swiglu,
npu_dequant_swiglu_quant, grouped_matmul, moe_distribute_dispatch, moe_distribute_combine,
grouped_matmul_swiglu_quant_v2}.py).  "Meta" implementations carry the shape rules; "CUDA" implementations
launch the sm_100a kernels on the current stream.  There is deliberately no CPU implementation: calling an
op on CPU tensors raises from the dispatcher, and argument combinations outside the path raise
NotImplementedError instead of falling back.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Optional

import torch
from torch.library import Library

from . import _lib, ep

# c10::ScalarType integers used for dtype arguments (python/torchair/ge/_ge_graph.py:215-270).
_ST = {1: torch.int8, 3: torch.int32, 5: torch.float16, 6: torch.float32, 15: torch.bfloat16}
_ST_INV = {v: k for k, v in _ST.items()}

# npu_moe_init_routing has no expert-count argument; ids must lie below this bound (bins of the counting sort).
INIT_ROUTING_EXPERT_BOUND = 1024

_npu = Library("npu", "FRAGMENT")

_npu.define("npu_moe_init_routing(Tensor x, Tensor row_idx, Tensor expert_idx, int active_num) -> (Tensor, Tensor, Tensor)")
_npu.define("npu_dynamic_quant(Tensor input, *, Tensor? smooth_scales=None, Tensor? group_index=None, int? dst_type=None, "
            "str quant_mode=\"pertoken\", float dst_type_max=0.0) -> (Tensor, Tensor)")
_npu.define("npu_dynamic_quant_asymmetric(Tensor input, *, Tensor? smooth_scales=None, Tensor? group_index=None, "
            "int? dst_type=None, str quant_mode=\"pertoken\", float dst_type_max=0.0) -> (Tensor, Tensor, Tensor)")
_npu.define("npu_swiglu(Tensor self, int dim=-1) -> Tensor")
_npu.define("npu_dequant_swiglu_quant(Tensor x, *, Tensor? weight_scale=None, Tensor? activation_scale=None, "
            "Tensor? bias=None, Tensor? quant_scale=None, Tensor? quant_offset=None, Tensor? group_index=None, "
            "bool activate_left=False, int quant_mode=0, int? dst_type=None, int? round_mode=None, "
            "int? activate_dim=None, int swiglu_mode=0, float clamp_limit=7.0, float glu_alpha=1.702, "
            "float glu_bias=1.0) -> (Tensor, Tensor)")
_GMM_TAIL = ("Tensor[]? activation_input=None, Tensor[]? activation_quant_scale=None, "
             "Tensor[]? activation_quant_offset=None, int? split_item=0, int? group_type=-1, int? group_list_type=0, "
             "int? act_type=0, int[]? tuning_config=None, int? output_dtype=None, int? x_dtype=None, "
             "int? weight_dtype=None, int? scale_dtype=None, int? per_token_scale_dtype=None) -> Tensor[]")
_GMM_HEAD = ("(Tensor[] x, Tensor[] weight, *, Tensor[]? bias=None, Tensor[]? scale=None, Tensor[]? offset=None, "
             "Tensor[]? antiquant_scale=None, Tensor[]? antiquant_offset=None, Tensor[]? per_token_scale=None, ")
_npu.define("npu_grouped_matmul" + _GMM_HEAD + "Tensor? group_list=None, " + _GMM_TAIL)
_npu.define("npu_grouped_matmul.List" + _GMM_HEAD + "int[]? group_list=None, " + _GMM_TAIL)
_npu.define("npu_grouped_matmul_swiglu_quant_v2(Tensor x, Tensor[] weight, Tensor[] weight_scale, Tensor x_scale, "
            "Tensor group_list, *, Tensor? smooth_scale=None, Tensor[]? weight_assist_matrix=None, Tensor? bias=None, "
            "int? dequant_mode=0, int? dequant_dtype=0, int? quant_mode=0, int? quant_dtype=1, int? group_list_type=0, "
            "int[]? tuning_config=None, int? x_dtype=None, int? weight_dtype=None, int? weight_scale_dtype=None, "
            "int? x_scale_dtype=None) -> (Tensor, Tensor)")
_npu.define("npu_grouped_matmul_finalize_routing(Tensor x, Tensor w, Tensor group_list, *, Tensor? scale=None, Tensor? bias=None, "
            "Tensor? offset=None, Tensor? pertoken_scale=None, Tensor? shared_input=None, Tensor? logit=None, "
            "Tensor? row_index=None, ScalarType? dtype=None, float? shared_input_weight=1.0, int? shared_input_offset=0, "
            "int? output_bs=0, int? group_list_type=1, int[]? tuning_config=None, int? x_dtype=None, int? w_dtype=None, "
            "int? scale_dtype=None, int? pertoken_scale_dtype=None) -> Tensor")
_npu.define("npu_moe_compute_expert_tokens(Tensor sorted_experts, int num_experts) -> Tensor")
_npu.define("npu_moe_gating_top_k_softmax(Tensor x, Tensor? finished=None, int k=1) -> (Tensor, Tensor, Tensor)")
_npu.define("npu_moe_gating_top_k_softmax_v2(Tensor x, *, int k=1, Tensor? finished=None, int? renorm=0, bool? output_softmax=False) "
            "-> (Tensor, Tensor, Tensor)")
_npu.define("npu_moe_gating_top_k(Tensor x, int k, *, Tensor? bias=None, int k_group=1, int group_count=1, int group_select_mode=0, "
            "int renorm=0, int norm_type=0, bool out_flag=False, float routed_scaling_factor=1.0, float eps=1e-20) "
            "-> (Tensor, Tensor, Tensor)")
_V2_DISPATCH = ("(Tensor x, Tensor expert_ids, str group_ep, int ep_world_size, int ep_rank_id, int moe_expert_num, *, "
                "Tensor? scales=None, Tensor? x_active_mask=None, Tensor? expert_scales=None, Tensor? elastic_info=None, "
                "Tensor? performance_info=None, str group_tp=\"\", int tp_world_size=0, int tp_rank_id=0, int expert_shard_type=0, "
                "int shared_expert_num=1, int shared_expert_rank_num=0, int quant_mode=0, int global_bs=0, "
                "int expert_token_nums_type=1, str comm_alg=\"\", int zero_expert_num=0, int copy_expert_num=0, "
                "int const_expert_num=0, int? y_dtype=None, int? x_dtype=None, int? scales_dtype=None) "
                "-> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
_npu.define("npu_moe_distribute_dispatch_v2" + _V2_DISPATCH)
_npu.define("npu_moe_distribute_combine_v2(Tensor expand_x, Tensor expert_ids, Tensor assist_info_for_combine, Tensor ep_send_counts, "
            "Tensor expert_scales, str group_ep, int ep_world_size, int ep_rank_id, int moe_expert_num, *, "
            "Tensor? tp_send_counts=None, Tensor? x_active_mask=None, Tensor? expand_scales=None, Tensor? shared_expert_x=None, "
            "Tensor? elastic_info=None, Tensor? ori_x=None, Tensor? const_expert_alpha_1=None, Tensor? const_expert_alpha_2=None, "
            "Tensor? const_expert_v=None, Tensor? performance_info=None, str group_tp=\"\", int tp_world_size=0, int tp_rank_id=0, "
            "int expert_shard_type=0, int shared_expert_num=1, int shared_expert_rank_num=0, int global_bs=0, "
            "int comm_quant_mode=0, str comm_alg=\"\", int zero_expert_num=0, int copy_expert_num=0, int const_expert_num=0) "
            "-> Tensor")
_npu.define("npu_moe_finalize_routing(Tensor expanded_permuted_rows, Tensor? skip1, Tensor? skip2, Tensor? bias, Tensor? scales, "
            "Tensor expanded_src_to_dst_row, Tensor? export_for_source_row, int? drop_pad_mode=0) -> Tensor")
_npu.define("npu_moe_init_routing_v2(Tensor x, Tensor expert_idx, *, Tensor? scale=None, Tensor? offset=None, int active_num=-1, "
            "int expert_capacity=-1, int expert_num=-1, int drop_pad_mode=0, int expert_tokens_num_type=0, "
            "bool expert_tokens_num_flag=False, int quant_mode=-1, int[]? active_expert_range=None, int row_idx_type=0, "
            "int? x_dtype=None) -> (Tensor, Tensor, Tensor, Tensor)")
_npu.define("npu_moe_distribute_dispatch(Tensor x, Tensor expert_ids, str group_ep, int ep_world_size, int ep_rank_id, "
            "int moe_expert_num, *, Tensor? scales=None, Tensor? x_active_mask=None, Tensor? expert_scales=None, "
            "str group_tp=\"\", int tp_world_size=0, int tp_rank_id=0, int expert_shard_type=0, int shared_expert_num=1, "
            "int shared_expert_rank_num=0, int quant_mode=0, int global_bs=0, int expert_token_nums_type=1) "
            "-> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
_npu.define("npu_moe_distribute_combine(Tensor expand_x, Tensor expert_ids, Tensor expand_idx, Tensor ep_send_counts, "
            "Tensor expert_scales, str group_ep, int ep_world_size, int ep_rank_id, int moe_expert_num, *, "
            "Tensor? tp_send_counts=None, Tensor? x_active_mask=None, Tensor? activation_scale=None, "
            "Tensor? weight_scale=None, Tensor? group_list=None, Tensor? expand_scales=None, Tensor? shared_expert_x=None, "
            "str group_tp=\"\", int tp_world_size=0, int tp_rank_id=0, int expert_shard_type=0, int shared_expert_num=1, "
            "int shared_expert_rank_num=0, int global_bs=0, int out_dtype=0, int comm_quant_mode=0, "
            "int group_list_type=0) -> Tensor")


# --------------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------------
def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _st(dtype: torch.dtype, what: str) -> int:
    if dtype not in _ST_INV:
        raise NotImplementedError(f"{what}: dtype {dtype} is outside the W8A8 MoE path")
    return _ST_INV[dtype]


def _workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)


def _only_none(op: str, **kwargs):
    for k, v in kwargs.items():
        if v is not None:
            raise NotImplementedError(f"{op}: argument `{k}` is outside the W8A8 MoE path and must be None")


def _only_default(op: str, **pairs):
    for k, (v, d) in pairs.items():
        if v != d:
            raise NotImplementedError(f"{op}: `{k}`={v!r} is outside the W8A8 MoE path (supported: {d!r})")


# --------------------------------------------------------------------------------------------------
# npu_moe_init_routing
# --------------------------------------------------------------------------------------------------
def _init_routing_meta(x, row_idx, expert_idx, active_num):
    if x.dim() != 2 or expert_idx.dim() != 2 or row_idx.shape != expert_idx.shape:
        raise RuntimeError("npu_moe_init_routing: x must be [T, H]; row_idx and expert_idx [T, K]")
    T, K = expert_idx.shape
    rows = min(T, active_num) * K
    return (x.new_empty((rows, x.shape[1])), expert_idx.new_empty((T * K,)), expert_idx.new_empty((T * K,)))


def _init_routing_cuda(x, row_idx, expert_idx, active_num):
    ex, eri, eei = _init_routing_meta(x, row_idx, expert_idx, active_num)
    if row_idx.dtype != torch.int32 or expert_idx.dtype != torch.int32:
        raise RuntimeError("npu_moe_init_routing: row_idx and expert_idx must be int32")
    T, K = expert_idx.shape
    x, row_idx, expert_idx = x.contiguous(), row_idx.contiguous(), expert_idx.contiguous()
    ws = _workspace(_lib.workspace_bytes("tab_moe_init_routing_workspace_bytes", T, K, INIT_ROUTING_EXPERT_BOUND), x.device)
    _lib.call("tab_moe_init_routing", _ptr(x), _st(x.dtype, "npu_moe_init_routing"), _ptr(row_idx), _ptr(expert_idx),
              T, K, x.shape[1], active_num, INIT_ROUTING_EXPERT_BOUND, _ptr(ex), _ptr(eri), _ptr(eei), _ptr(ws),
              ws.numel(), _stream(x))
    return ex, eri, eei


# --------------------------------------------------------------------------------------------------
# npu_dynamic_quant
# --------------------------------------------------------------------------------------------------
def _dynamic_quant_check(op, group_index, dst_type, quant_mode, dst_type_max):
    _only_none(op, group_index=group_index)
    if dst_type not in (None, 1):
        raise NotImplementedError(f"{op}: dst_type={dst_type} (only 1 = int8 is on the path)")
    _only_default(op, quant_mode=(quant_mode, "pertoken"), dst_type_max=(dst_type_max, 0.0))


def _dynamic_quant_meta(input, *, smooth_scales=None, group_index=None, dst_type=None, quant_mode="pertoken", dst_type_max=0.0):
    _dynamic_quant_check("npu_dynamic_quant", group_index, dst_type, quant_mode, dst_type_max)
    if input.dim() < 1:
        raise RuntimeError("npu_dynamic_quant: input must have at least one dimension")
    return (torch.empty(input.shape, dtype=torch.int8, device=input.device),
            torch.empty(input.shape[:-1], dtype=torch.float32, device=input.device))


def _dynamic_quant_cuda(input, *, smooth_scales=None, group_index=None, dst_type=None, quant_mode="pertoken", dst_type_max=0.0):
    y, scale = _dynamic_quant_meta(input, smooth_scales=smooth_scales, group_index=group_index, dst_type=dst_type,
                                   quant_mode=quant_mode, dst_type_max=dst_type_max)
    x = input.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    if smooth_scales is not None:
        if smooth_scales.dtype != x.dtype or smooth_scales.numel() != cols:
            raise RuntimeError("npu_dynamic_quant: smooth_scales must be [H] of the input dtype")
        smooth_scales = smooth_scales.contiguous()
    _lib.call("tab_dynamic_quant", _ptr(x), _st(x.dtype, "npu_dynamic_quant"), _ptr(smooth_scales), rows, cols,
              _ptr(y), _ptr(scale), _stream(x))
    return y, scale


def _dynamic_quant_asym(input, *, smooth_scales=None, group_index=None, dst_type=None, quant_mode="pertoken", dst_type_max=0.0):
    raise NotImplementedError("npu_dynamic_quant_asymmetric is outside the W8A8 MoE path (symmetric per-token int8 only)")


# --------------------------------------------------------------------------------------------------
# npu_swiglu
# --------------------------------------------------------------------------------------------------
def _swiglu_meta(self, dim=-1):
    d = dim if dim >= 0 else dim + self.dim()
    if d < 0 or d >= self.dim() or self.shape[d] % 2:
        raise RuntimeError("npu_swiglu: the split dimension must exist and be even")
    shape = list(self.shape)
    shape[d] //= 2
    return self.new_empty(shape)


def _swiglu_cuda(self, dim=-1):
    out = _swiglu_meta(self, dim)
    d = dim if dim >= 0 else dim + self.dim()
    if d != self.dim() - 1:
        raise NotImplementedError("npu_swiglu: only the last dimension can be split on this path")
    x = self.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    _lib.call("tab_swiglu", _ptr(x), _st(x.dtype, "npu_swiglu"), rows, cols, _ptr(out), _stream(x))
    return out


# --------------------------------------------------------------------------------------------------
# npu_dequant_swiglu_quant
# --------------------------------------------------------------------------------------------------
def _dsq_meta(x, *, weight_scale=None, activation_scale=None, bias=None, quant_scale=None, quant_offset=None,
              group_index=None, activate_left=False, quant_mode=0, dst_type=None, round_mode=None, activate_dim=None,
              swiglu_mode=0, clamp_limit=7.0, glu_alpha=1.702, glu_bias=1.0):
    # shape rule of python/torchair/_contrib/custom_torch_ops/auto_register_custom_torch_ops.py:121-156
    activate_dim = -1 if activate_dim is None else activate_dim
    select = activate_dim if activate_dim >= 0 else activate_dim + x.dim()
    if x.dim() <= 1:
        raise RuntimeError("x dim should larger than 1")
    if select < 0 or select >= x.dim():
        raise RuntimeError("activate dim should less than x dim")
    if x.size(select) % 2 != 0:
        raise RuntimeError("x last dim should be even")
    if quant_mode not in (0, 1):
        raise RuntimeError("quant_mode only support 0 or 1, but got " + str(quant_mode))
    y_size = [x.size(i) // 2 if i == select else x.size(i) for i in range(x.dim())]
    return (torch.empty(y_size, dtype=torch.int8, device=x.device),
            torch.empty(y_size[:-1], dtype=torch.float32, device=x.device))


def _dsq_cuda(x, *, weight_scale=None, activation_scale=None, bias=None, quant_scale=None, quant_offset=None,
              group_index=None, activate_left=False, quant_mode=0, dst_type=None, round_mode=None, activate_dim=None,
              swiglu_mode=0, clamp_limit=7.0, glu_alpha=1.702, glu_bias=1.0):
    op = "npu_dequant_swiglu_quant"
    y, scale = _dsq_meta(x, quant_mode=quant_mode, activate_dim=activate_dim)
    _only_none(op, bias=bias, quant_scale=quant_scale, quant_offset=quant_offset)
    if quant_mode != 1:
        raise NotImplementedError(f"{op}: only quant_mode=1 (dynamic) is on the path")
    if dst_type not in (None, 1) or round_mode not in (None, 0) or swiglu_mode != 0:
        raise NotImplementedError(f"{op}: only int8 output, rint rounding and swiglu_mode=0 are on the path")
    if activate_dim not in (None, -1, x.dim() - 1):
        raise NotImplementedError(f"{op}: only the last dimension can be split on this path")
    if x.dtype != torch.int32:
        raise NotImplementedError(f"{op}: x must be int32 accumulators on this path")
    x = x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols
    ws_groups = 0
    if weight_scale is not None:
        if weight_scale.dtype != torch.float32 or weight_scale.shape[-1] != cols:
            raise RuntimeError(f"{op}: weight_scale must be fp32 [.., {cols}]")
        weight_scale = weight_scale.contiguous()
        ws_groups = weight_scale.numel() // cols
    if activation_scale is not None:
        if activation_scale.dtype != torch.float32 or activation_scale.numel() != rows:
            raise RuntimeError(f"{op}: activation_scale must be fp32 with one value per row")
        activation_scale = activation_scale.contiguous()
    ngroups = 0
    if group_index is not None:
        group_index = group_index.to(torch.int64).contiguous()
        ngroups = group_index.numel()
    _lib.call("tab_dequant_swiglu_quant", _ptr(x), _ptr(weight_scale), ws_groups, _ptr(activation_scale), _ptr(group_index),
              ngroups, int(bool(activate_left)), rows, cols, _ptr(y), _ptr(scale), _stream(x))
    return y, scale


# --------------------------------------------------------------------------------------------------
# npu_grouped_matmul (W8A8) and the packed-weight cache
# --------------------------------------------------------------------------------------------------
_packed_cache = {}


def clear_weight_cache() -> None:
    """Drops the cached K-major relayouts of expert weights (call after freeing or replacing weights)."""
    _packed_cache.clear()


def packed_weight(weight: torch.Tensor) -> torch.Tensor:
    """int8 [E, Kd, N] -> cached int8 [E, N, Kd] (the K-major operand layout the tcgen05 descriptors read).

    One-off per weight tensor.  The cache entry is tied to the life of the weight's storage (it is dropped by a
    finaliser when the storage is freed, so a new tensor that reuses the address never sees a stale relayout)
    and to the tensor's version counter (an in-place update of the weights triggers a fresh relayout).
    """
    if weight.dim() == 3 and weight.shape[1] > 1 and weight.shape[2] > 1 and weight.permute(0, 2, 1).is_contiguous():
        # already K-major underneath: an [E, Kd, N] view of a packed [E, N, Kd] buffer, as use_internal_format_weight(...,
        # release_original=True) leaves it.  Nothing to relay out, nothing to cache.
        return weight.permute(0, 2, 1)
    storage = weight.untyped_storage()
    ident = (storage._cdata, weight.storage_offset(), tuple(weight.shape), tuple(weight.stride()))
    hit = _packed_cache.get(ident)
    if hit is not None and hit[0] == weight._version:
        return hit[1]
    w = weight.contiguous()
    E, Kd, N = w.shape
    out = torch.empty((E, N, Kd), dtype=torch.int8, device=w.device)
    _lib.call("tab_prepack_weight_i8", _ptr(w), E, Kd, N, _ptr(out), _stream(w))
    if w.is_cuda and torch.cuda.is_current_stream_capturing():
        # first use inside a CUDA-graph capture: the relayout becomes part of that graph and its result lives in the graph's
        # pool, valid only after a replay, so it must not serve later eager calls (pack ahead with
        # use_internal_format_weight, or run once eagerly, to keep the relayout out of the graph)
        return out
    if hit is None:
        weakref.finalize(storage, _packed_cache.pop, ident, None)
    _packed_cache[ident] = (weight._version, out)
    return out


def _gmm_common_check(op, x, weight, split_item, group_type, group_list, act_type):
    if len(x) != 1 or len(weight) != 1:
        raise NotImplementedError(f"{op}: exactly one x and one weight tensor (split_item 2/3 form) are on the path")
    xs, w = x[0], weight[0]
    if xs.dtype != torch.int8 or w.dtype != torch.int8:
        raise NotImplementedError(f"{op}: only int8 x int8 (W8A8) is on the path, got {xs.dtype} x {w.dtype}")
    if xs.dim() != 2 or w.dim() != 3 or xs.shape[1] != w.shape[1]:
        raise RuntimeError(f"{op}: x must be [M, K] and weight [E, K, N]")
    if split_item not in (2, 3):
        raise NotImplementedError(f"{op}: split_item must be 2 or 3 (single output tensor)")
    if group_type != 0:
        raise NotImplementedError(f"{op}: group_type must be 0 (groups split the M axis)")
    if group_list is None:
        raise RuntimeError(f"{op}: group_list is required")
    if act_type not in (None, 0):
        raise NotImplementedError(f"{op}: act_type must be 0")
    return xs, w


def _expected_rows(tuning_config) -> int:
    """First element of tuning_config = the rows a group is expected to hold (0 / absent = unknown).  The converters forward
    the list to the IR attribute of the same name without defining it (grouped_matmul.py:245,361); decision: expected
    rows per group, used only to choose the kernel orientation and tile width."""
    if tuning_config is None or len(tuning_config) == 0:
        return 0
    v = int(tuning_config[0])
    return v if v > 0 else 0


def _gmm_out_dtype(output_dtype):
    # converter grouped_matmul.py:178-195: fp16 -> 0, bf16 -> 1, int32 -> 2; int8 is rejected
    if output_dtype is None:
        raise NotImplementedError("npu_grouped_matmul: output_dtype is required for int8 inputs (3, 5 or 15)")
    if output_dtype not in (3, 5, 15):
        raise ValueError(f"output_dtype should be int32, float16 or bfloat16, but got {output_dtype}")
    return _ST[output_dtype]


def _gmm_meta(x, weight, *, bias=None, scale=None, offset=None, antiquant_scale=None, antiquant_offset=None,
              per_token_scale=None, group_list=None, activation_input=None, activation_quant_scale=None,
              activation_quant_offset=None, split_item=0, group_type=-1, group_list_type=0, act_type=0,
              tuning_config=None, output_dtype=None, x_dtype=None, weight_dtype=None, scale_dtype=None,
              per_token_scale_dtype=None):
    xs, w = _gmm_common_check("npu_grouped_matmul", x, weight, split_item, group_type, group_list, act_type)
    return [torch.empty((xs.shape[0], w.shape[2]), dtype=_gmm_out_dtype(output_dtype), device=xs.device)]


def _gmm_cuda(x, weight, *, bias=None, scale=None, offset=None, antiquant_scale=None, antiquant_offset=None,
              per_token_scale=None, group_list=None, activation_input=None, activation_quant_scale=None,
              activation_quant_offset=None, split_item=0, group_type=-1, group_list_type=0, act_type=0,
              tuning_config=None, output_dtype=None, x_dtype=None, weight_dtype=None, scale_dtype=None,
              per_token_scale_dtype=None):
    op = "npu_grouped_matmul"
    xs, w = _gmm_common_check(op, x, weight, split_item, group_type, group_list, act_type)
    for name, v in (("offset", offset), ("antiquant_scale", antiquant_scale),
                    ("antiquant_offset", antiquant_offset), ("activation_input", activation_input),
                    ("activation_quant_scale", activation_quant_scale), ("activation_quant_offset", activation_quant_offset)):
        if v is not None and len(v) > 0:
            raise NotImplementedError(f"{op}: `{name}` is outside the W8A8 MoE path")
    _only_none(op, x_dtype=x_dtype, weight_dtype=weight_dtype, scale_dtype=scale_dtype, per_token_scale_dtype=per_token_scale_dtype)
    out_dt = _gmm_out_dtype(output_dtype)
    M, Kd = xs.shape
    E, _, N = w.shape
    if isinstance(group_list, (list, tuple)):
        group_list = torch.tensor(list(group_list), dtype=torch.int64, device=xs.device)
    if group_list.numel() != E:
        raise RuntimeError(f"{op}: group_list must have one entry per expert ({E})")
    group_list = group_list.to(torch.int64).contiguous()
    sc = scale[0] if scale is not None and len(scale) else None
    pts = per_token_scale[0] if per_token_scale is not None and len(per_token_scale) else None
    bs = bias[0] if bias is not None and len(bias) else None
    if bs is not None:
        # the int8 mode takes an int32 bias (converter grouped_matmul.py:258-262), added to the accumulators
        if bs.dtype != torch.int32 or bs.numel() != E * N:
            raise NotImplementedError(f"{op}: bias must be int32 [E, N] for int8 inputs")
        bs = bs.contiguous()
    if out_dt != torch.int32:
        if sc is not None:
            if sc.dtype not in (torch.float32, torch.bfloat16) or sc.numel() != E * N:
                raise NotImplementedError(f"{op}: scale must be float32 or bfloat16 [E, N] on this path")
            sc = sc.float().contiguous()          # a bfloat16 scale is an exact float32 value
        if pts is not None:
            if pts.dtype != torch.float32 or pts.numel() != M:
                raise RuntimeError(f"{op}: per_token_scale must be fp32 [M]")
            pts = pts.contiguous()
    xs = xs.contiguous()
    wp = packed_weight(w)
    # rows outside every group are left unwritten: with expert parallelism x is sized for the worst case and most of
    # it is an unused tail, which nothing downstream reads
    y = torch.empty((M, N), dtype=out_dt, device=xs.device)
    _lib.call("tab_grouped_matmul_w8a8", _ptr(xs), _ptr(wp), _ptr(sc), _ptr(pts), _ptr(bs), _ptr(group_list), int(group_list_type or 0),
              M, Kd, N, E, _ST_INV[out_dt], _ptr(y), _expected_rows(tuning_config), _stream(xs))
    return [y]


def _gmm_sq_meta(x, weight, weight_scale, x_scale, group_list, *, smooth_scale=None, weight_assist_matrix=None, bias=None,
                 dequant_mode=0, dequant_dtype=0, quant_mode=0, quant_dtype=1, group_list_type=0, tuning_config=None,
                 x_dtype=None, weight_dtype=None, weight_scale_dtype=None, x_scale_dtype=None):
    if len(weight) != 1 or weight[0].dim() != 3 or x.dim() != 2 or weight[0].shape[2] % 2:
        raise RuntimeError("npu_grouped_matmul_swiglu_quant_v2: x [M, K], one weight [E, K, 2*I]")
    M, I = x.shape[0], weight[0].shape[2] // 2
    return (torch.empty((M, I), dtype=torch.int8, device=x.device), torch.empty((M,), dtype=torch.float32, device=x.device))


def _gmm_sq_cuda(x, weight, weight_scale, x_scale, group_list, *, smooth_scale=None, weight_assist_matrix=None, bias=None,
                 dequant_mode=0, dequant_dtype=0, quant_mode=0, quant_dtype=1, group_list_type=0, tuning_config=None,
                 x_dtype=None, weight_dtype=None, weight_scale_dtype=None, x_scale_dtype=None):
    op = "npu_grouped_matmul_swiglu_quant_v2"
    yq, ys = _gmm_sq_meta(x, weight, weight_scale, x_scale, group_list)
    _only_none(op, smooth_scale=smooth_scale, bias=bias, x_dtype=x_dtype, weight_dtype=weight_dtype,
               weight_scale_dtype=weight_scale_dtype, x_scale_dtype=x_scale_dtype)
    if weight_assist_matrix is not None and len(weight_assist_matrix):
        raise NotImplementedError(f"{op}: weight_assist_matrix is outside the W8A8 MoE path")
    _only_default(op, dequant_mode=(dequant_mode or 0, 0), quant_mode=(quant_mode or 0, 0), quant_dtype=(quant_dtype or 1, 1))
    return fused_gate_up(x, weight[0], weight_scale[0], x_scale, group_list, int(group_list_type or 0), True, yq, ys,
                         _expected_rows(tuning_config))


def fused_gate_up(x, w, w_scale, x_scale, group_list, group_list_type, activate_left, yq=None, ys=None, expected_rows=0):
    """gate_up grouped GEMM + dequant + SwiGLU + per-row int8 requant in one call (two kernels)."""
    if x.dtype != torch.int8 or w.dtype != torch.int8:
        raise NotImplementedError("fused gate_up: only int8 x int8 (W8A8) is on the path")
    M, Kd = x.shape
    E, _, N2 = w.shape
    I = N2 // 2
    if yq is None:
        yq = torch.empty((M, I), dtype=torch.int8, device=x.device)
        ys = torch.empty((M,), dtype=torch.float32, device=x.device)
    if w_scale.dtype != torch.float32 or w_scale.numel() != E * N2 or x_scale.dtype != torch.float32 or x_scale.numel() != M:
        raise RuntimeError("fused gate_up: weight_scale must be fp32 [E, 2*I] and x_scale fp32 [M]")
    if group_list.numel() != E:
        raise RuntimeError(f"fused gate_up: group_list must have one entry per expert ({E})")
    group_list = group_list.to(torch.int64).contiguous()
    x, w_scale, x_scale = x.contiguous(), w_scale.contiguous(), x_scale.contiguous()
    wp = packed_weight(w)
    ws = _workspace(_lib.workspace_bytes("tab_grouped_matmul_swiglu_quant_workspace_bytes", M, I), x.device)
    _lib.call("tab_grouped_matmul_swiglu_quant", _ptr(x), _ptr(wp), _ptr(w_scale), _ptr(x_scale), _ptr(group_list),
              group_list_type, M, Kd, I, E, int(bool(activate_left)), _ptr(yq), _ptr(ys), _ptr(ws), ws.numel(), int(expected_rows),
              _stream(x))
    return yq, ys


# --------------------------------------------------------------------------------------------------
# npu_grouped_matmul_finalize_routing (converter grouped_matmul_finalize_routing.py:57-133): down GEMM + weighted
# scatter-add into fp32 token rows, optionally on top of the shared experts' rows
# --------------------------------------------------------------------------------------------------
def _gmm_fr_meta(x, w, group_list, *, scale=None, bias=None, offset=None, pertoken_scale=None, shared_input=None, logit=None,
                 row_index=None, dtype=None, shared_input_weight=1.0, shared_input_offset=0, output_bs=0, group_list_type=1,
                 tuning_config=None, x_dtype=None, w_dtype=None, scale_dtype=None, pertoken_scale_dtype=None):
    op = "npu_grouped_matmul_finalize_routing"
    if x.dim() != 2 or w.dim() != 3 or w.shape[1] != x.shape[1]:
        raise RuntimeError(f"{op}: x [M, K] and w [E, K, N] expected, got {tuple(x.shape)} and {tuple(w.shape)}")
    if dtype is not None and dtype != torch.float32:
        raise RuntimeError(f"Not supported output dtype is {dtype}")      # the converter's own message
    rows = int(output_bs or 0) or x.shape[0]
    return torch.empty((rows, w.shape[2]), dtype=torch.float32, device=x.device)


def _gmm_fr_cuda(x, w, group_list, *, scale=None, bias=None, offset=None, pertoken_scale=None, shared_input=None, logit=None,
                 row_index=None, dtype=None, shared_input_weight=1.0, shared_input_offset=0, output_bs=0, group_list_type=1,
                 tuning_config=None, x_dtype=None, w_dtype=None, scale_dtype=None, pertoken_scale_dtype=None):
    op = "npu_grouped_matmul_finalize_routing"
    y = _gmm_fr_meta(x, w, group_list, dtype=dtype, output_bs=output_bs)
    _only_none(op, offset=offset, x_dtype=x_dtype, w_dtype=w_dtype, scale_dtype=scale_dtype, pertoken_scale_dtype=pertoken_scale_dtype)
    if x.dtype != torch.int8 or w.dtype != torch.int8:
        raise NotImplementedError(f"{op}: only int8 x int8 (W8A8) is on the path")
    M, Kd = x.shape
    E, _, N = w.shape
    if group_list.numel() != E:
        raise RuntimeError(f"{op}: group_list must have one entry per expert ({E})")
    if row_index is None or row_index.numel() != M or row_index.dtype not in (torch.int32, torch.int64):
        raise RuntimeError(f"{op}: row_index must be int32 or int64 [M]")
    if scale is not None:
        if scale.numel() != E * N:
            raise RuntimeError(f"{op}: scale must be [E, N]")
        scale = scale.to(torch.float32).contiguous()
    if bias is not None:
        if bias.numel() != E * N:
            raise RuntimeError(f"{op}: bias must be [E, N]")
        bias = bias.to(torch.bfloat16).contiguous()
    for name, t in (("pertoken_scale", pertoken_scale), ("logit", logit)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != M):
            raise RuntimeError(f"{op}: {name} must be fp32 [M]")
    shared_rows = 0
    if shared_input is not None:
        if shared_input.dim() != 2 or shared_input.shape[1] != N or shared_input.dtype != torch.bfloat16:
            raise RuntimeError(f"{op}: shared_input must be bfloat16 [rows, N]")
        shared_rows = shared_input.shape[0]
        shared_input = shared_input.contiguous()
    group_list = group_list.to(torch.int64).contiguous()
    x, row_index = x.contiguous(), row_index.contiguous()
    pertoken_scale = None if pertoken_scale is None else pertoken_scale.contiguous()
    logit = None if logit is None else logit.contiguous()
    wp = packed_weight(w)
    ws = _workspace(_lib.workspace_bytes("tab_grouped_matmul_finalize_routing_workspace_bytes", M, N), x.device)
    _lib.call("tab_grouped_matmul_finalize_routing", _ptr(x), _ptr(wp), _ptr(scale), _ptr(bias), _ptr(pertoken_scale),
              _ptr(group_list), int(1 if group_list_type is None else group_list_type), M, Kd, N, E, _ptr(shared_input), shared_rows,
              float(1.0 if shared_input_weight is None else shared_input_weight), int(shared_input_offset or 0), _ptr(logit),
              _ptr(row_index), 3 if row_index.dtype == torch.int32 else 4, y.shape[0], _ptr(y), _ptr(ws), ws.numel(),
              _expected_rows(tuning_config), _stream(x))
    return y


def fused_down_combine(hq, w2, s2, hs, group_list, group_list_type, expert_ids, expand_idx, ep_send_counts, expert_scales,
                       group_ep, ep_world_size, ep_rank_id, moe_expert_num, shared_expert_x=None, out_dtype=torch.bfloat16,
                       expected_rows=0):
    """Down projection + npu_moe_distribute_combine as one step.

    With more than one rank on the peer-memory transport the grouped GEMM's epilogue stores every output row straight
    into the return buffer of the rank that sent the token (NVLink stores from inside the GEMM kernel, tile by tile), so
    the transfer overlaps the GEMM and no [rows, H] tensor or copy kernel exists.  Otherwise it is the two operators
    one after the other.  Results are identical either way.
    """
    R = int(ep_world_size)
    od = 15 if out_dtype == torch.bfloat16 else 5
    if R == 1 or ep.transport_of(group_ep, hq.is_cuda) != "peer":
        y = torch.ops.npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=group_list, split_item=2,
                                             group_type=0, group_list_type=group_list_type, output_dtype=od,
                                             tuning_config=[int(expected_rows)])[0]
        return torch.ops.npu.npu_moe_distribute_combine(y, expert_ids, expand_idx, ep_send_counts, expert_scales, group_ep, R,
                                                        ep_rank_id, moe_expert_num, shared_expert_x=shared_expert_x)
    if hq.dtype != torch.int8 or w2.dtype != torch.int8:
        raise NotImplementedError("fused down + combine: only int8 x int8 (W8A8) is on the path")
    ep.check_combine_args(hq, expert_ids, expert_scales, R, ep_rank_id, moe_expert_num, None, None, None, None, 0, 0, 0, 0, 0, 0)
    M, Kd = hq.shape
    E_l, _, N = w2.shape
    if s2.dtype != torch.float32 or s2.numel() != E_l * N or hs.dtype != torch.float32 or hs.numel() != M or group_list.numel() != E_l:
        raise RuntimeError("fused down + combine: scale must be fp32 [E_l, H], per-token scale fp32 [M], group_list [E_l]")
    hq, s2, hs = hq.contiguous(), s2.contiguous(), hs.contiguous()
    gl = group_list.to(torch.int64).contiguous()
    wp = packed_weight(w2)

    def produce_rows(row_dst):
        _lib.call("tab_grouped_matmul_w8a8_scatter", _ptr(hq), _ptr(wp), _ptr(s2), _ptr(hs), _ptr(gl), int(group_list_type), M, Kd, N,
                  E_l, od, _ptr(row_dst), int(expected_rows), _stream(hq))

    return ep.combine_from_producer(ep.CudaKernels, produce_rows, M, N, out_dtype, expert_ids, expand_idx, ep_send_counts,
                                    expert_scales, group_ep, R, ep_rank_id, moe_expert_num, shared_expert_x)


def _device(device):
    return torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)


def gmm_status(device=None) -> int:
    """Synchronises the current stream and returns the GEMM kernels' device status word: 0, or the code of the first
    bounded wait that gave up since the last gmm_status_reset (raises RuntimeError in that case)."""
    dev = _device(device)
    with torch.cuda.device(dev):
        st = ctypes.c_int(0)
        _lib.call("tab_gmm_status", ctypes.byref(st), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        return int(st.value)


def gmm_status_reset(device=None) -> None:
    """Clears the GEMM kernels' sticky status word (synchronises the current stream)."""
    dev = _device(device)
    with torch.cuda.device(dev):
        _lib.call("tab_gmm_status_reset", ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))


def routing_status(device=None) -> int:
    """Synchronises the current stream, returns and clears the routing kernels' status word: bit 0 = an expert id
    outside the valid range was clamped, bit 1 = a row_idx value outside [0, T*K) was skipped.  Does not raise."""
    dev = _device(device)
    with torch.cuda.device(dev):
        st = ctypes.c_int(0)
        rc = _lib.load().tab_routing_status(ctypes.byref(st), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        if rc != 0 and st.value == 0:
            raise RuntimeError(f"tab_routing_status failed ({rc}): {_lib.last_error()}")
        return int(st.value)


def check_status(device=None) -> None:
    """Raises RuntimeError if, since the last check, a bounded wait inside a GEMM or a peer-memory exchange gave up or
    a routing kernel met an index out of range.  Synchronises the device: call it where the step synchronises anyway."""
    st = routing_status(device)
    if st:
        raise RuntimeError(f"routing kernels met indices out of range (status {st}): " + _lib.last_error())
    dev = _device(device)
    with torch.cuda.device(dev):
        st_ = ctypes.c_int(0)
        rc = _lib.load().tab_gmm_status(ctypes.byref(st_), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        if rc != 0:
            msg = _lib.last_error()
            if st_.value:
                gmm_status_reset(dev)
            raise RuntimeError(f"grouped GEMM status {st_.value}: {msg}")
        _lib.call("tab_quant_status", ctypes.byref(st_), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    st = ep.peer_status()
    if st:
        raise RuntimeError(f"peer-memory exchange status {st}: a flag wait ran out of time or a slot overflowed")



# --------------------------------------------------------------------------------------------------
# operators next to the path: expert token counts, gating, finalize, routing with built-in quantisation
# --------------------------------------------------------------------------------------------------
def _cet_meta(sorted_experts, num_experts):
    if sorted_experts.dim() != 1 or num_experts <= 0:
        raise RuntimeError("npu_moe_compute_expert_tokens: sorted_experts must be 1-D and num_experts positive")
    return torch.empty((num_experts,), dtype=torch.int32, device=sorted_experts.device)


def _cet_cuda(sorted_experts, num_experts):
    out = _cet_meta(sorted_experts, num_experts)
    if sorted_experts.dtype != torch.int32:
        raise RuntimeError("npu_moe_compute_expert_tokens: sorted_experts must be int32")
    se = sorted_experts.contiguous()
    _lib.call("tab_moe_compute_expert_tokens", _ptr(se), se.numel(), num_experts, _ptr(out), _stream(se))
    return out


def _gating_meta(x, finished=None, k=1):
    if x.dim() != 2 or k < 1 or k > x.shape[1]:
        raise RuntimeError("npu_moe_gating_top_k_softmax: x must be [tokens, experts] and 1 <= k <= experts")
    T = x.shape[0]
    return (x.new_empty((T, k)), torch.empty((T, k), dtype=torch.int32, device=x.device),
            torch.empty((T, k), dtype=torch.int32, device=x.device))


def _finished_mask(op, finished, tokens):
    if finished is None:
        return None
    if finished.dtype != torch.bool or finished.numel() != tokens:
        raise RuntimeError(f"{op}: finished must be bool [tokens]")
    return finished.contiguous()


def _gating_cuda(x, finished=None, k=1):
    y, ei, ri = _gating_meta(x, finished, k)
    fin = _finished_mask("npu_moe_gating_top_k_softmax", finished, x.shape[0])
    xc = x.contiguous()
    _lib.call("tab_moe_gating_top_k_softmax", _ptr(xc), _st(x.dtype, "npu_moe_gating_top_k_softmax"), _ptr(fin), x.shape[0],
              x.shape[1], k, _ptr(y), _ptr(ei), _ptr(ri), _stream(xc))
    return y, ei, ri


def _gating_v2_meta(x, *, k=1, finished=None, renorm=0, output_softmax=False):
    if x.dim() != 2 or k < 1 or k > x.shape[1]:
        raise RuntimeError("npu_moe_gating_top_k_softmax_v2: x must be [tokens, experts] and 1 <= k <= experts")
    T, E = x.shape
    full = bool(output_softmax) and not renorm        # the softmax over all experts exists only without renormalisation
    return (x.new_empty((T, k)), torch.empty((T, k), dtype=torch.int32, device=x.device),
            torch.empty((T, E) if full else (0,), dtype=torch.float32, device=x.device))


def _gating_v2_cuda(x, *, k=1, finished=None, renorm=0, output_softmax=False):
    op = "npu_moe_gating_top_k_softmax_v2"
    y, ei, sm = _gating_v2_meta(x, k=k, renorm=renorm, output_softmax=output_softmax)
    fin = _finished_mask(op, finished, x.shape[0])
    if (renorm or 0) not in (0, 1):
        raise RuntimeError(f"{op}: renorm must be 0 or 1")
    xc = x.contiguous()
    _lib.call("tab_moe_gating_top_k", _ptr(xc), None, _ptr(fin), _st(x.dtype, op), x.shape[0], x.shape[1], k, 1, 1, 0, 2 if renorm else 0,
              1.0, 0.0, _ptr(y), _ptr(ei), _ptr(sm) if sm.numel() else None, _stream(xc))
    return y, ei, sm


def _gating2_meta(x, k, *, bias=None, k_group=1, group_count=1, group_select_mode=0, renorm=0, norm_type=0, out_flag=False,
                  routed_scaling_factor=1.0, eps=1e-20):
    # shape rule of python/torchair/_contrib/custom_torch_ops/auto_register_custom_torch_ops.py:69-79
    if x.dim() != 2 or k < 1 or k > x.shape[1]:
        raise RuntimeError("npu_moe_gating_top_k: x must be [tokens, experts] and 1 <= k <= experts")
    return (x.new_empty((x.size(0), k)), x.new_empty((x.size(0), k), dtype=torch.int32),
            x.new_empty((x.size(0), x.size(1)), dtype=torch.float32))


def _gating2_cuda(x, k, *, bias=None, k_group=1, group_count=1, group_select_mode=0, renorm=0, norm_type=0, out_flag=False,
                  routed_scaling_factor=1.0, eps=1e-20):
    op = "npu_moe_gating_top_k"
    y, ei, out = _gating2_meta(x, k)
    if renorm not in (0, 1) or (renorm == 1 and norm_type != 0):
        raise NotImplementedError(f"{op}: renorm must be 0, or 1 together with norm_type 0 (softmax renormalised over the k)")
    xc = x.contiguous()
    if bias is not None:
        if bias.dtype != x.dtype or bias.numel() != x.shape[1]:
            raise RuntimeError(f"{op}: bias must be [experts] of the dtype of x")
        bias = bias.contiguous()
    _lib.call("tab_moe_gating_top_k", _ptr(xc), _ptr(bias), None, _st(x.dtype, op), x.shape[0], x.shape[1], k, k_group, group_count,
              int(group_select_mode), 2 if renorm == 1 else int(norm_type), float(routed_scaling_factor), float(eps), _ptr(y),
              _ptr(ei), _ptr(out), _stream(xc))
    return y, ei, out


_comm_alg_seen = set()


def _comm_alg_hint(op, comm_alg):
    """comm_alg names one of the vendor's exchange algorithms.  Here the transport of the group decides how rows move
    (register_ep_group), so the hint changes nothing; it is accepted and reported once per value."""
    if not isinstance(comm_alg, str):
        raise RuntimeError(f"{op}: comm_alg must be a string")
    if comm_alg and comm_alg not in _comm_alg_seen:
        _comm_alg_seen.add(comm_alg)
        import logging
        logging.getLogger("torchair").warning("%s: comm_alg=%r has no effect on B200; the group's transport moves the rows", op, comm_alg)


_elastic_checked = {}


def _check_elastic_info(op, elastic_info, R):
    """elastic_info (moe_distribute_dispatch_v2.py:16,72): int32 [4 + 2 * ep_world_size].  Decision: entry 0 says whether the
    group runs in a shrunk (elastic) state; the rest is the rank table of that state.  Only the full group is served here
    (entry 0 == 0); a shrunk group is re-registered under a new name with register_ep_group instead.  The contents are read
    once per tensor version, outside CUDA-graph capture (a host read)."""
    if elastic_info is None:
        return
    if elastic_info.dtype != torch.int32 or elastic_info.numel() != 4 + 2 * R:
        raise RuntimeError(f"{op}: elastic_info must be int32 with 4 + 2 * ep_world_size = {4 + 2 * R} entries")
    key = (elastic_info.data_ptr(), elastic_info._version)
    if key in _elastic_checked or (elastic_info.is_cuda and torch.cuda.is_current_stream_capturing()):
        return
    if int(elastic_info.reshape(-1)[0].item()) != 0:
        raise NotImplementedError(f"{op}: a shrunk (elastic) group is not served through elastic_info; register the surviving "
                                  "ranks as a new group")
    if len(_elastic_checked) > 64:
        _elastic_checked.clear()
    _elastic_checked[key] = True


def _check_performance_info(op, performance_info, R):
    """performance_info (moe_distribute_dispatch_v2.py:17,73): int64 [ep_world_size] in which the vendor kernel accumulates how
    long it waited for each rank.  Accepted and left unchanged: the waits of this implementation are device-side and
    report through the status words."""
    if performance_info is not None and (performance_info.dtype != torch.int64 or performance_info.numel() != R):
        raise RuntimeError(f"{op}: performance_info must be int64 [ep_world_size]")


def _special_counts(op, zero_expert_num, copy_expert_num, const_expert_num):
    for n in (zero_expert_num, copy_expert_num, const_expert_num):
        if not isinstance(n, int) or n < 0:
            raise RuntimeError(f"{op}: zero_expert_num, copy_expert_num and const_expert_num must be non-negative integers")
    return zero_expert_num + copy_expert_num + const_expert_num


def _dispatch_v2(impl, is_meta):
    def fn(x, expert_ids, group_ep, ep_world_size, ep_rank_id, moe_expert_num, *, scales=None, x_active_mask=None,
           expert_scales=None, elastic_info=None, performance_info=None, group_tp="", tp_world_size=0, tp_rank_id=0,
           expert_shard_type=0, shared_expert_num=1, shared_expert_rank_num=0, quant_mode=0, global_bs=0,
           expert_token_nums_type=1, comm_alg="", zero_expert_num=0, copy_expert_num=0, const_expert_num=0, y_dtype=None,
           x_dtype=None, scales_dtype=None):
        op = "npu_moe_distribute_dispatch_v2"
        _only_none(op, x_dtype=x_dtype, scales_dtype=scales_dtype)
        _comm_alg_hint(op, comm_alg)
        _check_performance_info(op, performance_info, ep_world_size)
        special = _special_counts(op, zero_expert_num, copy_expert_num, const_expert_num)
        if y_dtype is not None:
            # the converter's rule (moe_distribute_dispatch_v2.py:60-64): int8 unless quant_mode is 0, then the dtype of x;
            # y_dtype may restate that, it cannot ask for another element type here
            want = 1 if quant_mode != 0 else _ST_INV.get(x.dtype)
            if y_dtype != want:
                raise NotImplementedError(f"{op}: y_dtype={y_dtype} differs from the output type of quant_mode={quant_mode} ({want})")
        kw = dict(scales=scales, x_active_mask=x_active_mask, expert_scales=expert_scales, group_tp=group_tp,
                  tp_world_size=tp_world_size, tp_rank_id=tp_rank_id, expert_shard_type=expert_shard_type,
                  shared_expert_num=shared_expert_num, shared_expert_rank_num=shared_expert_rank_num, quant_mode=quant_mode,
                  global_bs=global_bs, expert_token_nums_type=expert_token_nums_type)
        if not is_meta:
            _check_elastic_info(op, elastic_info, ep_world_size)
            kw["_special"] = special
        return impl(x, expert_ids, group_ep, ep_world_size, ep_rank_id, moe_expert_num, **kw)
    return fn


def _combine_v2(impl, is_meta):
    def fn(expand_x, expert_ids, assist_info_for_combine, ep_send_counts, expert_scales, group_ep, ep_world_size, ep_rank_id,
           moe_expert_num, *, tp_send_counts=None, x_active_mask=None, expand_scales=None, shared_expert_x=None, elastic_info=None,
           ori_x=None, const_expert_alpha_1=None, const_expert_alpha_2=None, const_expert_v=None, performance_info=None,
           group_tp="", tp_world_size=0, tp_rank_id=0, expert_shard_type=0, shared_expert_num=1, shared_expert_rank_num=0,
           global_bs=0, comm_quant_mode=0, comm_alg="", zero_expert_num=0, copy_expert_num=0, const_expert_num=0):
        op = "npu_moe_distribute_combine_v2"
        _comm_alg_hint(op, comm_alg)
        _check_performance_info(op, performance_info, ep_world_size)
        specials = _special_counts(op, zero_expert_num, copy_expert_num, const_expert_num)
        T, H = expert_ids.shape[0], expand_x.shape[1]
        if copy_expert_num + const_expert_num > 0 and (ori_x is None or tuple(ori_x.shape) != (T, H)):
            raise RuntimeError(f"{op}: copy and constant experts need ori_x [T, H]")
        if const_expert_num > 0:
            for name, t in (("const_expert_alpha_1", const_expert_alpha_1), ("const_expert_alpha_2", const_expert_alpha_2),
                            ("const_expert_v", const_expert_v)):
                if t is None or tuple(t.shape) != (const_expert_num, H):
                    raise RuntimeError(f"{op}: {name} must be [const_expert_num, H]")
        kw = dict(tp_send_counts=tp_send_counts, x_active_mask=x_active_mask, expand_scales=expand_scales,
                  shared_expert_x=shared_expert_x, group_tp=group_tp, tp_world_size=tp_world_size, tp_rank_id=tp_rank_id,
                  expert_shard_type=expert_shard_type, shared_expert_num=shared_expert_num,
                  shared_expert_rank_num=shared_expert_rank_num, global_bs=global_bs, comm_quant_mode=comm_quant_mode)
        if not is_meta:
            _check_elastic_info(op, elastic_info, ep_world_size)
            if specials > 0:
                kw["_special"] = {"expert_ids": expert_ids, "E": moe_expert_num, "zero": zero_expert_num, "copy": copy_expert_num,
                                  "const": const_expert_num, "ori_x": ori_x, "alpha_1": const_expert_alpha_1,
                                  "alpha_2": const_expert_alpha_2, "const_v": const_expert_v}
        return impl(expand_x, expert_ids, assist_info_for_combine, ep_send_counts, expert_scales, group_ep, ep_world_size,
                    ep_rank_id, moe_expert_num, **kw)
    return fn


def _finalize_meta(expanded_permuted_rows, skip1, skip2, bias, scales, expanded_src_to_dst_row, export_for_source_row,
                   drop_pad_mode=0):
    rows = expanded_permuted_rows
    if rows.dim() != 2 or expanded_src_to_dst_row.dim() != 1:
        raise RuntimeError("npu_moe_finalize_routing: rows must be [T*K, H] and expanded_src_to_dst_row 1-D")
    if scales is not None:
        T = scales.shape[0]
    elif skip1 is not None:
        T = skip1.shape[0]
    else:
        T = expanded_src_to_dst_row.numel()
    return rows.new_empty((T, rows.shape[1]))


def _finalize_cuda(expanded_permuted_rows, skip1, skip2, bias, scales, expanded_src_to_dst_row, export_for_source_row,
                   drop_pad_mode=0):
    op = "npu_moe_finalize_routing"
    out = _finalize_meta(expanded_permuted_rows, skip1, skip2, bias, scales, expanded_src_to_dst_row, export_for_source_row)
    if drop_pad_mode not in (None, 0):
        raise NotImplementedError(f"{op}: only drop_pad_mode=0 (dropless) is on the path")
    rows = expanded_permuted_rows.contiguous()
    T, H = out.shape
    K = expanded_src_to_dst_row.numel() // T
    if K * T != expanded_src_to_dst_row.numel() or expanded_src_to_dst_row.dtype != torch.int32:
        raise RuntimeError(f"{op}: expanded_src_to_dst_row must be int32 with K*T entries")
    for name, t in (("skip1", skip1), ("skip2", skip2), ("bias", bias)):
        if t is not None and t.dtype != rows.dtype:
            raise RuntimeError(f"{op}: {name} must have the dtype of the rows")
    if bias is not None and (export_for_source_row is None or export_for_source_row.dtype != torch.int32):
        raise RuntimeError(f"{op}: bias needs int32 export_for_source_row [T, K]")
    sc = None if scales is None else scales.to(torch.float32).contiguous()
    c = lambda t: None if t is None else t.contiguous()
    skip1, skip2, bias, efr = c(skip1), c(skip2), c(bias), c(export_for_source_row)
    _lib.call("tab_moe_finalize_routing", _ptr(rows), _st(rows.dtype, op), _ptr(skip1), _ptr(skip2), _ptr(bias), _ptr(sc),
              _ptr(expanded_src_to_dst_row.contiguous()), _ptr(efr), T, K, H, _ptr(out), _stream(rows))
    return out


def _irv2_check(x, expert_idx, scale, offset, active_num, expert_capacity, expert_num, drop_pad_mode, quant_mode,
                active_expert_range, x_dtype):
    """Returns (expert_lo, expert_hi, rows of expanded_x, active_rows)."""
    op = "npu_moe_init_routing_v2"
    if x.dim() != 2 or expert_idx.dim() != 2 or x.shape[0] != expert_idx.shape[0]:
        raise RuntimeError(f"{op}: x must be [T, H] and expert_idx [T, K]")
    _only_none(op, offset=offset, x_dtype=x_dtype)
    if expert_num <= 0:
        raise RuntimeError(f"{op}: expert_num must be given")
    if drop_pad_mode != 0 or expert_capacity not in (-1, 0):
        raise NotImplementedError(f"{op}: only the dropless mode is on the path")
    if quant_mode not in (-1, 1):
        raise NotImplementedError(f"{op}: quant_mode must be -1 (none) or 1 (per-token dynamic int8)")
    lo, hi = 0, expert_num
    if active_expert_range is not None and len(active_expert_range):
        if len(active_expert_range) != 2:
            raise RuntimeError(f"{op}: active_expert_range must be [expert_start, expert_end]")
        lo, hi = int(active_expert_range[0]), int(active_expert_range[1])
        if not (0 <= lo < hi <= expert_num):
            raise RuntimeError(f"{op}: active_expert_range [{lo}, {hi}) must lie inside [0, expert_num = {expert_num})")
    T, K = expert_idx.shape
    M, H = T * K, x.shape[1]
    active_rows = int(active_num) if active_num is not None and 0 < active_num < M else 0
    if scale is not None:
        if scale.dtype != torch.float32:
            raise RuntimeError(f"{op}: scale must be float32")
        if quant_mode == -1 and scale.numel() != T:
            raise RuntimeError(f"{op}: without quantisation scale holds one value per token ({T})")
        if quant_mode == 1 and (scale.numel() not in (H, (hi - lo) * H) or scale.shape[-1] != H):
            raise RuntimeError(f"{op}: with dynamic quantisation scale must be [{hi - lo}, {H}] or [1, {H}]")
    return lo, hi, (active_rows or M), active_rows


def _irv2_meta(x, expert_idx, *, scale=None, offset=None, active_num=-1, expert_capacity=-1, expert_num=-1, drop_pad_mode=0,
               expert_tokens_num_type=0, expert_tokens_num_flag=False, quant_mode=-1, active_expert_range=None, row_idx_type=0,
               x_dtype=None):
    lo, hi, rows, _ = _irv2_check(x, expert_idx, scale, offset, active_num, expert_capacity, expert_num, drop_pad_mode, quant_mode,
                                  active_expert_range, x_dtype)
    M = expert_idx.numel()
    dev = x.device
    return (torch.empty((rows, x.shape[1]), dtype=torch.int8 if quant_mode == 1 else x.dtype, device=dev),
            torch.empty((M,), dtype=torch.int32, device=dev), torch.empty((hi - lo,), dtype=torch.int64, device=dev),
            torch.empty((M,), dtype=torch.float32, device=dev))


def _irv2_cuda(x, expert_idx, *, scale=None, offset=None, active_num=-1, expert_capacity=-1, expert_num=-1, drop_pad_mode=0,
               expert_tokens_num_type=0, expert_tokens_num_flag=False, quant_mode=-1, active_expert_range=None, row_idx_type=0,
               x_dtype=None):
    lo, hi, rows, active_rows = _irv2_check(x, expert_idx, scale, offset, active_num, expert_capacity, expert_num, drop_pad_mode,
                                            quant_mode, active_expert_range, x_dtype)
    ex, eri, tokens, esc = _irv2_meta(x, expert_idx, scale=scale, offset=offset, active_num=active_num,
                                      expert_capacity=expert_capacity, expert_num=expert_num, drop_pad_mode=drop_pad_mode,
                                      quant_mode=quant_mode, active_expert_range=active_expert_range, x_dtype=x_dtype)
    if expert_idx.dtype != torch.int32 or x.dtype not in (torch.bfloat16, torch.float16):
        raise NotImplementedError("npu_moe_init_routing_v2: x must be bfloat16/float16 and expert_idx int32")
    T, K = expert_idx.shape
    xc, ic = x.contiguous(), expert_idx.contiguous()
    sc = None if scale is None else scale.contiguous()
    scale_rows = 0 if sc is None else (T if quant_mode == -1 else sc.numel() // x.shape[1])
    nbytes = _lib.workspace_bytes("tab_moe_dispatch_pack_workspace_bytes", T, K, hi - lo) + 4 * (T * K + hi - lo) + 1024
    ws = _workspace(nbytes, x.device)
    _lib.call("tab_moe_init_routing_v2", _ptr(xc), _st(x.dtype, "npu_moe_init_routing_v2"), _ptr(ic), T, K, x.shape[1], lo, hi,
              quant_mode, int(expert_tokens_num_type), int(row_idx_type), active_rows, _ptr(sc), scale_rows, _ptr(ex), _ptr(eri),
              _ptr(tokens), _ptr(esc), _ptr(ws), ws.numel(), _stream(xc))
    return ex, eri, tokens, esc


# --------------------------------------------------------------------------------------------------
# npu_moe_distribute_dispatch / combine
# --------------------------------------------------------------------------------------------------
def _dispatch_meta(x, expert_ids, group_ep, ep_world_size, ep_rank_id, moe_expert_num, *, scales=None, x_active_mask=None,
                   expert_scales=None, group_tp="", tp_world_size=0, tp_rank_id=0, expert_shard_type=0, shared_expert_num=1,
                   shared_expert_rank_num=0, quant_mode=0, global_bs=0, expert_token_nums_type=1):
    ep.check_dispatch_args(x, expert_ids, ep_world_size, ep_rank_id, moe_expert_num, scales, x_active_mask, tp_world_size,
                           expert_shard_type, shared_expert_rank_num, quant_mode, global_bs, expert_token_nums_type)
    T, K = expert_ids.shape
    R = ep_world_size
    E_l = moe_expert_num // R
    A = ep.dispatch_rows(T, R, moe_expert_num, K, global_bs)
    dev = x.device
    return (torch.empty((A, x.shape[1]), dtype=torch.int8 if quant_mode == 2 else x.dtype, device=dev),
            torch.empty((A,), dtype=torch.float32, device=dev),
            torch.empty((T * K,), dtype=torch.int32, device=dev),
            torch.empty((E_l,), dtype=torch.int64, device=dev),
            torch.empty((E_l * R,), dtype=torch.int32, device=dev),
            torch.empty((max(tp_world_size, 1),), dtype=torch.int32, device=dev),
            torch.empty((A,), dtype=torch.float32, device=dev))


def _dispatch_cuda(x, expert_ids, group_ep, ep_world_size, ep_rank_id, moe_expert_num, *, scales=None, x_active_mask=None,
                   expert_scales=None, group_tp="", tp_world_size=0, tp_rank_id=0, expert_shard_type=0, shared_expert_num=1,
                   shared_expert_rank_num=0, quant_mode=0, global_bs=0, expert_token_nums_type=1, _special=0):
    ep.check_dispatch_args(x, expert_ids, ep_world_size, ep_rank_id, moe_expert_num, scales, x_active_mask, tp_world_size,
                           expert_shard_type, shared_expert_rank_num, quant_mode, global_bs, expert_token_nums_type)
    return ep.dispatch(ep.CudaKernels, x, expert_ids, group_ep, ep_world_size, ep_rank_id, moe_expert_num, quant_mode,
                       expert_token_nums_type, max(tp_world_size, 1), x_active_mask, scales, _special, global_bs)


def _combine_meta(expand_x, expert_ids, expand_idx, ep_send_counts, expert_scales, group_ep, ep_world_size, ep_rank_id,
                  moe_expert_num, *, tp_send_counts=None, x_active_mask=None, activation_scale=None, weight_scale=None,
                  group_list=None, expand_scales=None, shared_expert_x=None, group_tp="", tp_world_size=0, tp_rank_id=0,
                  expert_shard_type=0, shared_expert_num=1, shared_expert_rank_num=0, global_bs=0, out_dtype=0,
                  comm_quant_mode=0, group_list_type=0):
    ep.check_combine_args(expand_x, expert_ids, expert_scales, ep_world_size, ep_rank_id, moe_expert_num, x_active_mask,
                          activation_scale, weight_scale, group_list, tp_world_size, expert_shard_type,
                          shared_expert_rank_num, global_bs, out_dtype, comm_quant_mode)
    return expand_x.new_empty((expert_ids.shape[0], expand_x.shape[1]))


def _combine_cuda(expand_x, expert_ids, expand_idx, ep_send_counts, expert_scales, group_ep, ep_world_size, ep_rank_id,
                  moe_expert_num, *, tp_send_counts=None, x_active_mask=None, activation_scale=None, weight_scale=None,
                  group_list=None, expand_scales=None, shared_expert_x=None, group_tp="", tp_world_size=0, tp_rank_id=0,
                  expert_shard_type=0, shared_expert_num=1, shared_expert_rank_num=0, global_bs=0, out_dtype=0,
                  comm_quant_mode=0, group_list_type=0, _special=None):
    ep.check_combine_args(expand_x, expert_ids, expert_scales, ep_world_size, ep_rank_id, moe_expert_num, x_active_mask,
                          activation_scale, weight_scale, group_list, tp_world_size, expert_shard_type,
                          shared_expert_rank_num, global_bs, out_dtype, comm_quant_mode)
    return ep.combine(ep.CudaKernels, expand_x, expert_ids, expand_idx, ep_send_counts, expert_scales, group_ep,
                      ep_world_size, ep_rank_id, moe_expert_num, shared_expert_x, x_active_mask, _special)


for _name, _meta, _cuda in (
        ("npu_moe_init_routing", _init_routing_meta, _init_routing_cuda),
        ("npu_dynamic_quant", _dynamic_quant_meta, _dynamic_quant_cuda),
        ("npu_swiglu", _swiglu_meta, _swiglu_cuda),
        ("npu_dequant_swiglu_quant", _dsq_meta, _dsq_cuda),
        ("npu_grouped_matmul", _gmm_meta, _gmm_cuda),
        ("npu_grouped_matmul.List", _gmm_meta, _gmm_cuda),
        ("npu_grouped_matmul_swiglu_quant_v2", _gmm_sq_meta, _gmm_sq_cuda),
        ("npu_grouped_matmul_finalize_routing", _gmm_fr_meta, _gmm_fr_cuda),
        ("npu_moe_compute_expert_tokens", _cet_meta, _cet_cuda),
        ("npu_moe_gating_top_k_softmax", _gating_meta, _gating_cuda),
        ("npu_moe_finalize_routing", _finalize_meta, _finalize_cuda),
        ("npu_moe_gating_top_k", _gating2_meta, _gating2_cuda),
        ("npu_moe_gating_top_k_softmax_v2", _gating_v2_meta, _gating_v2_cuda),
        ("npu_moe_init_routing_v2", _irv2_meta, _irv2_cuda),
        ("npu_moe_distribute_dispatch", _dispatch_meta, _dispatch_cuda),
        ("npu_moe_distribute_combine", _combine_meta, _combine_cuda)):
    _npu.impl(_name, _meta, "Meta")
    _npu.impl(_name, _cuda, "CUDA")
_npu.impl("npu_dynamic_quant_asymmetric", _dynamic_quant_asym, "CompositeExplicitAutograd")
# the second-generation dispatch / combine operators share the kernels: special experts are dropped from the exchange and
# evaluated by the combine; elastic_info and performance_info are accepted (see _check_elastic_info)
_npu.impl("npu_moe_distribute_dispatch_v2", _dispatch_v2(_dispatch_meta, True), "Meta")
_npu.impl("npu_moe_distribute_dispatch_v2", _dispatch_v2(_dispatch_cuda, False), "CUDA")
_npu.impl("npu_moe_distribute_combine_v2", _combine_v2(_combine_meta, True), "Meta")
_npu.impl("npu_moe_distribute_combine_v2", _combine_v2(_combine_cuda, False), "CUDA")

OP_NAMES = ["npu_moe_init_routing", "npu_dynamic_quant", "npu_dynamic_quant_asymmetric", "npu_swiglu",
            "npu_dequant_swiglu_quant", "npu_grouped_matmul", "npu_grouped_matmul_swiglu_quant_v2",
            "npu_moe_distribute_dispatch", "npu_moe_distribute_combine", "npu_moe_compute_expert_tokens",
            "npu_moe_gating_top_k_softmax", "npu_moe_finalize_routing", "npu_moe_init_routing_v2", "npu_moe_gating_top_k",
            "npu_moe_distribute_dispatch_v2", "npu_moe_distribute_combine_v2", "npu_grouped_matmul_finalize_routing",
            "npu_moe_gating_top_k_softmax_v2"]
