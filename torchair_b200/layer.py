"""The quantised expert-parallel MoE layer as a composition of torch.ops.npu.* calls.

This is the op sequence that serving stacks built on the reference emit for a W8A8 MoE feed-forward block
(each op is one converter under python/torchair/_ge_concrete_graph/ge_converter/custom): dispatch with per-token
int8 quantisation -> gate_up grouped matmul -> dequant + SwiGLU + requant -> down grouped matmul -> combine.
With ep_world_size == 1 no collective runs.
"""
from __future__ import annotations

import torch

from . import ops  # noqa: F401  (registers torch.ops.npu.*)


def moe_layer(x, expert_ids, expert_scales, w1, s1, w2, s2, *, group_ep: str = "", ep_world_size: int = 1,
              ep_rank_id: int = 0, moe_expert_num: int = None, fused: bool = True, after_dispatch=None):
    """x [T, H] bf16; expert_ids int32 [T, K]; expert_scales fp32 [T, K]; w1 int8 [E_l, H, 2I]; s1 fp32 [E_l, 2I];
    w2 int8 [E_l, I, H]; s2 fp32 [E_l, H] (this rank's experts).  Returns [T, H] bf16.

    fused=True issues gate_up + SwiGLU + requant as npu_grouped_matmul_swiglu_quant_v2 and, with more than one rank, the
    down projection together with the combine; fused=False issues the int32 grouped matmul, npu_dequant_swiglu_quant,
    the down grouped matmul and the combine separately (what the FX fusion passes rewrite).

    after_dispatch: optional callable without arguments, called once the dispatch has been enqueued.  A caller that has
    work of its own to run beside the layer (transfers for the next step on other streams, say) forks it there: next to
    the expert GEMMs it disturbs the step less than next to the latency-bound exchange at the step's start.
    """
    npu = torch.ops.npu
    R = ep_world_size
    E = moe_expert_num if moe_expert_num is not None else w1.shape[0] * R
    # rows an expert is expected to receive (all ranks' copies spread over all experts): the tiling hint of the grouped
    # matmuls.  With R > 1 the dispatch output is sized for the worst case, so the row count of `ex` says little.
    tune = [max(1, -(-x.shape[0] * expert_ids.shape[1] * R // E))]
    ex, xs, expand_idx, nums, ep_recv, _tp, _es = npu.npu_moe_distribute_dispatch(
        x, expert_ids, group_ep, R, ep_rank_id, E, quant_mode=2, expert_token_nums_type=1)
    if after_dispatch is not None:
        after_dispatch()
    if fused:
        hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(ex, [w1], [s1], xs, nums, group_list_type=1, tuning_config=tune)
    else:
        h32 = npu.npu_grouped_matmul([ex], [w1], group_list=nums, split_item=2, group_type=0, group_list_type=1,
                                     output_dtype=3, tuning_config=tune)[0]
        hq, hs = npu.npu_dequant_swiglu_quant(h32, weight_scale=s1, activation_scale=xs, group_index=nums,
                                              activate_left=True, quant_mode=1)
    if fused and R > 1 and not torch.compiler.is_compiling():
        # down GEMM and combine in one step: over peer memory the GEMM's epilogue stores its rows into the senders'
        # return buffers (a compiled graph gets the same rewrite from the FX pass of the backend)
        return ops.fused_down_combine(hq, w2, s2, hs, nums, 1, expert_ids, expand_idx, ep_recv, expert_scales, group_ep, R,
                                      ep_rank_id, E, out_dtype=x.dtype, expected_rows=tune[0])
    y = npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=nums, split_item=2,
                               group_type=0, group_list_type=1, output_dtype=15 if x.dtype == torch.bfloat16 else 5,
                               tuning_config=tune)[0]
    return npu.npu_moe_distribute_combine(y, expert_ids, expand_idx, ep_recv, expert_scales, group_ep, R, ep_rank_id, E)
