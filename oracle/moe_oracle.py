"""CPU oracle for the W8A8 expert-parallel MoE path (TEST INFRASTRUCTURE, not product code).

Only tests, the smoke check and the benchmark's CPU-baseline legs may import this module; the
shipped ops never call it and have no CPU fallback.

PARITY UNPINNED: the reference (Ascend/torchair) contains no arithmetic for these ops -- each is a
converter that lowers ``torch.ops.npu.<op>`` to one graph-IR node whose kernel is a closed vendor
binary, and none of the reference's tests pins a numerical result for them.  What the reference does
pin (op names, argument order, defaults, dtypes, output arity, a few shape rules) is checked by the
conformance tests.  The value semantics below follow the IR prototypes' doc comments and the
benchmark description (scale = amax/127, round-half-even, clamp +-127, per-channel weight scales,
per-token activation scales), evaluated in eager torch on CPU.  Every function cites the reference
file:line whose contract it restates; choices the reference leaves open are marked "decision".

Reference anchors (paths inside the reference project):
  python/torchair/_ge_concrete_graph/ge_converter/custom/moe_init_routing.py:10-21
  python/torchair/_ge_concrete_graph/ge_converter/custom/npu_dynamic_quant.py:8-40
  python/torchair/_ge_concrete_graph/ge_converter/custom/npu_swiglu.py:8-14
  python/torchair/_ge_concrete_graph/ge_converter/custom/npu_dequant_swiglu_quant.py:5-64
  python/torchair/_ge_concrete_graph/ge_converter/custom/grouped_matmul.py:210-365
  python/torchair/_ge_concrete_graph/ge_converter/custom/moe_distribute_dispatch.py:4-45
  python/torchair/_ge_concrete_graph/ge_converter/custom/moe_distribute_combine.py:4-60
  third_party/ascend/include/ops/op_proto/inc/experiment_ops.h:2111-2134, 3616-3652, 3764-3811
  third_party/ascend/include/ops/op_proto/inc/nn_quantize.h:28-54
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

# c10 ScalarType integers the converters compare dtype arguments against
# (python/torchair/ge/_ge_graph.py:215-270).
SCALAR_TYPE = {1: torch.int8, 3: torch.int32, 5: torch.float16, 6: torch.float32, 15: torch.bfloat16}


# --------------------------------------------------------------------------------------------------
# gating (not an op of the path; needed to make inputs)
# --------------------------------------------------------------------------------------------------
def gating_topk(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(logits fp32) -> top-k by stable descending sort -> weights renormalised to sum 1.

    Decision: ties keep the lower expert id first.  Returns (expert_ids int32 [T,k], weights fp32 [T,k]).
    """
    p = torch.softmax(logits.float(), dim=-1)
    order = torch.sort(p, dim=-1, descending=True, stable=True)
    ids = order.indices[:, :k].to(torch.int32)
    w = order.values[:, :k]
    w = w / w.sum(dim=-1, keepdim=True)
    return ids.contiguous(), w.contiguous()


# --------------------------------------------------------------------------------------------------
# npu_moe_init_routing
# --------------------------------------------------------------------------------------------------
def moe_init_routing(x: torch.Tensor, row_idx: torch.Tensor, expert_idx: torch.Tensor, active_num: int):
    """MoeInitRouting (experiment_ops.h:2111-2134; converter moe_init_routing.py:10-21).

    Stable sort of the T*K (token, k) pairs by expert id.  Decision: ties are ordered by the flattened
    index t*K+k.  With ``row_idx_sorted[i]`` the row_idx value of the i-th sorted pair:
      expanded_expert_idx[i]               = sorted expert id
      expanded_row_idx[row_idx_sorted[i]]  = i                      (inverse permutation)
      expanded_x[i]                        = x[row_idx_sorted[i] mod T]   for i < min(T, active_num)*K
    """
    T, K = expert_idx.shape
    flat_e = expert_idx.reshape(-1).to(torch.int64)
    order = torch.sort(flat_e, stable=True)
    sorted_e = order.values.to(torch.int32)
    row_sorted = row_idx.reshape(-1).to(torch.int64)[order.indices]
    expanded_row_idx = torch.empty(T * K, dtype=torch.int32)
    expanded_row_idx[row_sorted] = torch.arange(T * K, dtype=torch.int32)
    n_rows = min(T, active_num) * K
    expanded_x = x[(row_sorted % T)[:n_rows]].contiguous()
    return expanded_x, expanded_row_idx, sorted_e


# --------------------------------------------------------------------------------------------------
# npu_dynamic_quant
# --------------------------------------------------------------------------------------------------
def quantize_rows_f32(v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric int8 quantiser on fp32 values (DynamicQuant, nn_quantize.h:28-54).

    scale = amax(|v|)/127 (fp32 IEEE division); q = clamp(rint(v/scale), -127, 127) with IEEE division
    (not multiply-by-reciprocal) and round-half-even.  Decision: an all-zero row gives scale 0, q 0.
    """
    v = v.float()
    amax = v.abs().amax(dim=-1)
    scale = amax / 127.0
    safe = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = torch.round(v / safe.unsqueeze(-1))
    q = torch.where(scale.unsqueeze(-1) > 0, q, torch.zeros_like(q))
    q = q.clamp_(-127, 127).to(torch.int8)
    return q, scale


def dynamic_quant(x: torch.Tensor, smooth_scales: Optional[torch.Tensor] = None):
    """npu_dynamic_quant(input, *, smooth_scales=None, ...) -> (int8, fp32 scale of shape input.shape[:-1]).

    Converter npu_dynamic_quant.py:8-40.  smooth_scales ([H], same dtype as input) multiplies the input in
    fp32 before the row quantiser (decision: product taken in fp32, not rounded to the input dtype).
    """
    v = x.float()
    if smooth_scales is not None:
        v = v * smooth_scales.float()
    q, s = quantize_rows_f32(v.reshape(-1, x.shape[-1]))
    return q.reshape(x.shape), s.reshape(x.shape[:-1])


# --------------------------------------------------------------------------------------------------
# SwiGLU arithmetic: silu(a) * b with a deterministic exp
# --------------------------------------------------------------------------------------------------
# Decision: silu(a) * b = RN(RN(a * RN(1 / (1 + e))) * b), e = exp(-a) by a fixed sequence of correctly rounded fp32 operations
# (the same sequence as oracle/silu_exact.c and the CUDA kernels), so that CPU and GPU agree bit for bit.  A libm exp
# (what F.silu calls) differs between CPU and GPU in the last place, which would move int8 values after SwiGLU by one
# step at rounding ties.  SILU_IMPL = "libm" selects F.silu instead: the literal eager-torch formula, used by the timed
# CPU baseline and by the test that bounds the distance between the two forms (a few ulp).
SILU_IMPL = "exact"

_LOG2E = 1.4426950216293335          # RN32(log2(e)) = 0x1.715476p+0
_MAGIC = 12582912.0                  # 1.5 * 2^23
# 2^f on [-0.5, 0.5], degree 6 (c0..c6), fp32 values
_EXP2_COEF = (1.0, 0.6931471824645996, 0.24022646248340607, 0.05550328642129898, 0.009618489071726799,
              0.0013399930903688073, 0.0001534581242594868)


def _fma32(a: torch.Tensor, b, c) -> torch.Tensor:
    """Correctly rounded fp32 fused multiply-add RN32(a*b + c) of fp32 tensors (b, c may be Python floats that are fp32
    values).  The product is exact in fp64; the fp64 sum is rounded to odd (TwoSum gives the exact error; an inexact sum
    with an even last bit moves to its odd neighbour on the side of the error), after which rounding to fp32 cannot be
    a double rounding (53 >= 2*24 + 2 bits)."""
    a64 = a.double()
    b64 = b.double() if isinstance(b, torch.Tensor) else torch.tensor(b, dtype=torch.float64)
    c64 = c.double() if isinstance(c, torch.Tensor) else torch.tensor(c, dtype=torch.float64)
    p = a64 * b64
    s = p + c64
    bb = s - p
    err = (p - (s - bb)) + (c64 - bb)
    even = (s.view(torch.int64) & 1) == 0
    toward = torch.where(err > 0, torch.full_like(s, float("inf")), torch.full_like(s, float("-inf")))
    s = torch.where((err != 0) & even, torch.nextafter(s, toward), s)
    return s.float()


def _silu_mul_exact_torch(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """oracle/silu_exact.c op for op, in torch (fp32 tensors in, fp32 out)."""
    x = torch.fmin(torch.fmax(-a, torch.tensor(-80.0)), torch.tensor(80.0))
    nm = _fma32(x, _LOG2E, _MAGIC)
    n = nm - torch.tensor(_MAGIC, dtype=torch.float32)
    f = _fma32(x, _LOG2E, -n)
    p = torch.full_like(f, _EXP2_COEF[6])
    for c in _EXP2_COEF[5::-1]:
        p = _fma32(p, f, c)
    e = (p.view(torch.int32) + (n.to(torch.int32) << 23)).view(torch.float32)
    d = 1.0 + e
    y = torch.ones_like(d) / d          # IEEE reciprocal (tensor / tensor)
    return (a * y) * b


_silu_lib = None


def _load_silu_lib():
    """oracle/_build/libsilu_exact.so (gcc build of oracle/silu_exact.c) when it exists or can be built; else None."""
    global _silu_lib
    if _silu_lib is None:
        import ctypes
        import os
        import subprocess
        here = os.path.dirname(os.path.abspath(__file__))
        so = os.path.join(here, "_build", "libsilu_exact.so")
        src = os.path.join(here, "silu_exact.c")
        try:
            if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
                os.makedirs(os.path.dirname(so), exist_ok=True)
                subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", src, "-o", so, "-lm"],
                               check=True, capture_output=True)
            lib = ctypes.CDLL(so)
            lib.tab_oracle_silu_mul.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
            lib.tab_oracle_silu_mul.restype = None
            _silu_lib = lib
        except (OSError, subprocess.CalledProcessError):
            _silu_lib = False
    return _silu_lib or None


def build_c_oracle() -> bool:
    """Compiles the C restatement (called by the build step); True when the library is usable."""
    return _load_silu_lib() is not None


def silu_mul(a: torch.Tensor, b: torch.Tensor, impl: Optional[str] = None) -> torch.Tensor:
    """silu(a) * b on fp32 tensors.  impl: "exact" (C when built, else the torch restatement of the same operations),
    "exact_torch", or "libm" (F.silu); default SILU_IMPL."""
    impl = impl or SILU_IMPL
    a, b = a.float(), b.float()
    if impl == "libm":
        return F.silu(a) * b
    if impl == "exact":
        lib = _load_silu_lib()
        if lib is not None:
            a, b = torch.broadcast_tensors(a, b)
            a, b = a.contiguous(), b.contiguous()
            out = torch.empty_like(a)
            lib.tab_oracle_silu_mul(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel())
            return out
    elif impl != "exact_torch":
        raise ValueError(f"unknown SwiGLU implementation {impl!r}")
    return _silu_mul_exact_torch(a, b)


# --------------------------------------------------------------------------------------------------
# npu_swiglu
# --------------------------------------------------------------------------------------------------
def swiglu(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """SwiGlu (converter npu_swiglu.py:8-14): a, b = halves of x along dim; y = silu(a)*b in fp32, cast back."""
    a, b = torch.chunk(x.float(), 2, dim=dim)
    return silu_mul(a, b).to(x.dtype)


# --------------------------------------------------------------------------------------------------
# group bookkeeping
# --------------------------------------------------------------------------------------------------
def group_bounds(group_list: torch.Tensor, group_list_type: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(start, count) per group from a cumsum (type 0) or counts (type 1) list (grouped_matmul.py:306-361)."""
    g = group_list.to(torch.int64)
    if group_list_type == 0:
        ends = g
        starts = torch.cat([torch.zeros(1, dtype=torch.int64), g[:-1]])
        return starts, ends - starts
    if group_list_type == 1:
        ends = torch.cumsum(g, 0)
        return ends - g, g
    raise ValueError("group_list_type must be 0 (cumsum) or 1 (counts)")


def int8_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Exact int8 x int8 -> int32 product ([m,k] @ [k,n])."""
    if a.shape[0] == 0:
        return torch.zeros(0, b.shape[1], dtype=torch.int32)
    try:
        return torch._int_mm(a.contiguous(), b.contiguous())
    except RuntimeError:
        return a.to(torch.int32) @ b.to(torch.int32)


# --------------------------------------------------------------------------------------------------
# npu_grouped_matmul, W8A8 mode
# --------------------------------------------------------------------------------------------------
def grouped_matmul_w8a8(x: torch.Tensor, weight: torch.Tensor, scale: Optional[torch.Tensor],
                        per_token_scale: Optional[torch.Tensor], group_list: torch.Tensor,
                        group_list_type: int = 0, output_dtype: int = 15,
                        bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """GroupedMatmul, int8 x int8 (experiment_ops.h:3616-3652; converter grouped_matmul.py:210-361).

    Expert e owns rows [s_e, s_e+c_e).  acc = x[rows] @ weight[e] in exact int32 (+ int32 bias[e]).
    output_dtype 3 -> raw int32 accumulators; 15/5 -> bf16/fp16 of
    (float(acc) * per_token_scale[m]) * scale[e, n]   (decision: this order, no fused multiply-add).
    Rows not covered by any group are zero here; the CUDA path leaves them unwritten (with expert parallelism the
    input is sized for the worst case and the uncovered tail is never read), so tests compare covered rows only.
    """
    M = x.shape[0]
    E, Kd, N = weight.shape
    starts, counts = group_bounds(group_list, group_list_type)
    out_dt = SCALAR_TYPE[output_dtype]
    y = torch.zeros(M, N, dtype=out_dt)
    for e in range(E):
        s, c = int(starts[e]), int(counts[e])
        if c <= 0:
            continue
        acc = int8_matmul(x[s:s + c], weight[e])
        if bias is not None:
            acc = acc + bias[e].to(torch.int32)
        if out_dt == torch.int32:
            y[s:s + c] = acc
        else:
            v = acc.float()
            if per_token_scale is not None:
                v = v * per_token_scale[s:s + c].float().unsqueeze(-1)
            if scale is not None:
                v = v * scale[e].float().unsqueeze(0)
            y[s:s + c] = v.to(out_dt)
    return y


def grouped_matmul_finalize_routing(x, weight, group_list, scale=None, bias=None, pertoken_scale=None, shared_input=None,
                                    logit=None, row_index=None, shared_input_weight=1.0, shared_input_offset=0,
                                    output_bs=0, group_list_type=1):
    """GroupedMatmulFinalizeRouting, int8 x int8 (fusion_ops.h:640-725; converter
    grouped_matmul_finalize_routing.py:57-133, which sets output_bs = rows of x when it is 0).

    y fp32 [output_bs, N] starts at zero; rows [shared_input_offset, +rows of shared_input) are
    shared_input_weight * shared_input; then, in row order, every row m inside a group e adds
    logit[m] * ((float(acc[m]) * pertoken_scale[m]) * scale[e] + bias[e]) into y[row_index[m]]
    (decision: this operation order, every step rounded to fp32; the device adds in no fixed order).
    """
    M = x.shape[0]
    E, Kd, N = weight.shape
    rows = int(output_bs) or M
    y = torch.zeros(rows, N, dtype=torch.float32)
    if shared_input is not None:
        off = int(shared_input_offset)
        y[off:off + shared_input.shape[0]] = shared_input.float() * torch.tensor(shared_input_weight, dtype=torch.float32)
    starts, counts = group_bounds(group_list, group_list_type)
    for e in range(E):
        s, c = int(starts[e]), int(counts[e])
        if c <= 0:
            continue
        v = int8_matmul(x[s:s + c], weight[e]).float()
        if pertoken_scale is not None:
            v = v * pertoken_scale[s:s + c].float().unsqueeze(-1)
        if scale is not None:
            v = v * scale[e].float().unsqueeze(0)
        if bias is not None:
            v = v + bias[e].float().unsqueeze(0)
        if logit is not None:
            v = v * logit[s:s + c].float().unsqueeze(-1)
        idx = row_index[s:s + c].long()
        ok = (idx >= 0) & (idx < rows)
        y.index_add_(0, idx[ok], v[ok])
    return y


# --------------------------------------------------------------------------------------------------
# npu_dequant_swiglu_quant
# --------------------------------------------------------------------------------------------------
def dequant_swiglu_f32(x: torch.Tensor, weight_scale: Optional[torch.Tensor], activation_scale: Optional[torch.Tensor],
                       group_index: Optional[torch.Tensor], activate_left: bool) -> torch.Tensor:
    """fp32 value that the quantiser of DequantSwigluQuant sees (experiment_ops.h:3764-3811).

    v = (float(x) * activation_scale[m]) * weight_scale[g, n]; halves (left, right) of the last dim;
    activate_left True -> silu(left)*right, False -> silu(right)*left (experiment_ops.h:3782-3784).
    Decision: group_index holds per-group row COUNTS; rows beyond their sum produce zeros.
    """
    M = x.shape[0]
    v = x.float()
    if activation_scale is not None:
        v = v * activation_scale.float().reshape(M, 1)
    if weight_scale is not None:
        ws = weight_scale.float()
        if ws.dim() == 1 or ws.shape[0] == 1 and group_index is None:
            v = v * ws.reshape(1, -1)
        else:
            _, counts = group_bounds(group_index, 1)
            gid = torch.repeat_interleave(torch.arange(ws.shape[0]), counts.clamp(min=0))
            valid = gid.shape[0]
            vv = torch.zeros_like(v)
            vv[:valid] = v[:valid] * ws[gid]
            v = vv
    left, right = torch.chunk(v, 2, dim=-1)
    h = silu_mul(left, right) if activate_left else silu_mul(right, left)
    if group_index is not None:
        valid = int(group_bounds(group_index, 1)[1].clamp(min=0).sum())
        h[valid:] = 0
    return h


def dequant_swiglu_quant(x: torch.Tensor, weight_scale=None, activation_scale=None, group_index=None,
                         activate_left: bool = False, quant_mode: int = 0):
    """npu_dequant_swiglu_quant with quant_mode=1 (dynamic) -> (int8 [M, N/2], fp32 [M]).

    Converter npu_dequant_swiglu_quant.py:5-64; shape rule
    python/torchair/_contrib/custom_torch_ops/auto_register_custom_torch_ops.py:121-156.
    SwiGLU runs on the un-rounded fp32 dequantised value, then the row quantiser of dynamic_quant.
    """
    if quant_mode != 1:
        raise NotImplementedError("oracle covers the dynamic quant mode only")
    h = dequant_swiglu_f32(x, weight_scale, activation_scale, group_index, activate_left)
    return quantize_rows_f32(h)


# --------------------------------------------------------------------------------------------------
# combine, single rank (= finalize routing)
# --------------------------------------------------------------------------------------------------
def weighted_gather_sum(y: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor,
                        shared: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_k weights[t,k] * y[pos[t,k]] in fp32, ascending k, one rounding to y.dtype.

    Decision: product and sum are separate fp32 operations (no fused multiply-add); the optional shared
    expert row is added last in fp32.
    """
    T, K = weights.shape
    acc = torch.zeros(T, y.shape[1], dtype=torch.float32)
    for k in range(K):
        term = weights[:, k].float().unsqueeze(-1) * y[pos[:, k].long()].float()
        acc = term if k == 0 else acc + term
    if shared is not None:
        acc = acc + shared.float()
    return acc.to(y.dtype)


# --------------------------------------------------------------------------------------------------
# operators next to the path
# --------------------------------------------------------------------------------------------------
def moe_compute_expert_tokens(sorted_experts: torch.Tensor, num_experts: int) -> torch.Tensor:
    """MoeComputeExpertTokens (converter npu_moe_compute_expert_tokens.py:4-11): out[e] = #entries <= e, int32."""
    return torch.cumsum(torch.bincount(sorted_experts.long().clamp(min=0), minlength=num_experts)[:num_experts], 0).to(torch.int32)


def moe_gating_top_k_softmax(x: torch.Tensor, k: int, finished: Optional[torch.Tensor] = None):
    """MoeGatingTopKSoftmax (converter moe_gating_top_k_softmax.py:9-19; experiment_ops.h:2222-2241):
    y = k largest softmax probabilities (in x's dtype), expert_idx int32, row_idx[t, j] = j*T + t.
    Decisions: ties keep the lower expert id; a row whose `finished` flag is set reports expert_idx = number of experts
    (an id past the last expert) in every slot, its y and row_idx as usual."""
    T, E = x.shape
    p = torch.softmax(x.float(), dim=-1)
    order = torch.sort(p, dim=-1, descending=True, stable=True)
    row_idx = (torch.arange(k, dtype=torch.int32).view(1, k) * T + torch.arange(T, dtype=torch.int32).view(T, 1))
    idx = order.indices[:, :k].to(torch.int32)
    if finished is not None:
        idx = torch.where(finished.to(torch.bool).view(T, 1), torch.full_like(idx, E), idx)
    return order.values[:, :k].to(x.dtype), idx, row_idx.contiguous()


def moe_gating_top_k_softmax_v2(x: torch.Tensor, k: int, renorm: int = 0, output_softmax: bool = False,
                                finished: Optional[torch.Tensor] = None):
    """MoeGatingTopKSoftmaxV2 without `finished` (converter npu_moe_gating_top_k_softmax_v2.py:9-23;
    experiment_ops.h:2243-2265).  Decisions: renorm 0 -> y = the k largest softmax probabilities, softmax_result = the
    fp32 softmax over all experts when asked for; renorm 1 -> the same k probabilities divided by their sum taken in
    selection order (equal, up to rounding, to a softmax over the k largest logits).  Ties keep the lower expert id."""
    p = torch.softmax(x.float(), dim=-1)
    order = torch.sort(p, dim=-1, descending=True, stable=True)
    y = order.values[:, :k]
    if renorm:
        ysum = torch.zeros(x.shape[0])
        for j in range(k):
            ysum = ysum + y[:, j]
        y = y / ysum.unsqueeze(-1)
    full = p if (output_softmax and not renorm) else torch.empty(0, dtype=torch.float32)
    idx = order.indices[:, :k].to(torch.int32)
    if finished is not None:     # decision as in moe_gating_top_k_softmax: finished rows point past the experts
        idx = torch.where(finished.to(torch.bool).view(-1, 1), torch.full_like(idx, x.shape[1]), idx)
    return y.to(x.dtype), idx, full


def moe_gating_top_k(x, k, bias=None, k_group=1, group_count=1, group_select_mode=0, norm_type=0, routed_scaling_factor=1.0,
                     eps=1e-20):
    """MoeGatingTopK (converter npu_moe_gating_top_k.py:4-22; experiment_ops.h:3722-3761).  Decisions: scores = softmax
    (norm_type 0) or sigmoid (1) in fp32; the bias enters the selection only; groups are contiguous and scored by their
    maximum (mode 0) or the sum of their two largest selection scores (mode 1); ties keep the lower index; y = selected
    scores, for sigmoid divided by (their sum in selection order + eps), times routed_scaling_factor."""
    T, E = x.shape
    xf = x.float()
    sc = torch.softmax(xf, dim=-1) if norm_type == 0 else 1.0 / (1.0 + torch.exp(-xf))
    sel = sc + bias.float() if bias is not None else sc.clone()
    if group_count > 1:
        G = E // group_count
        g = sel.view(T, group_count, G)
        if group_select_mode == 0:
            gs = g.amax(dim=-1)
        else:
            top2 = torch.sort(g, dim=-1, descending=True, stable=True).values[..., :2]
            gs = top2[..., 0] + top2[..., 1]
        keep = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :k_group]
        mask = torch.zeros(T, group_count, dtype=torch.bool)
        mask.scatter_(1, keep, True)
        sel = torch.where(mask.unsqueeze(-1).expand(T, group_count, G).reshape(T, E), sel, torch.full_like(sel, float("-inf")))
    idx = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :k]
    y = torch.gather(sc, 1, idx)
    if norm_type == 1:
        ysum = torch.zeros(T)
        for j in range(k):
            ysum = ysum + y[:, j]
        y = y / (ysum + eps).unsqueeze(-1)
    y = y * routed_scaling_factor
    return y.to(x.dtype), idx.to(torch.int32), sc


def moe_finalize_routing(rows, skip1, skip2, bias, scales, src_to_dst, expert_for_row):
    """MoeFinalizeRouting, dropless (converter npu_moe_finalize_routing.py:21-41):
    out[t] = sum_k scales[t,k] * (rows[src_to_dst[k*T+t]] + bias[expert[t,k]]) + skip1[t] + skip2[t].
    Decision: fp32, ascending k, separate multiply and add, skips added last, one rounding."""
    T = scales.shape[0] if scales is not None else skip1.shape[0]
    K = src_to_dst.numel() // T
    acc = None
    for k in range(K):
        v = rows[src_to_dst[k * T:(k + 1) * T].long()].float()
        if bias is not None:
            v = v + bias[expert_for_row[:, k].long()].float()
        w = scales[:, k].float().unsqueeze(-1) if scales is not None else 1.0
        term = w * v
        acc = term if acc is None else acc + term
    if skip1 is not None:
        acc = acc + skip1.float()
    if skip2 is not None:
        acc = acc + skip2.float()
    return acc.to(rows.dtype)


def moe_init_routing_v2(x, expert_idx, expert_num, quant_mode=-1, expert_tokens_num_type=0, row_idx_type=0,
                        active_expert_range=None, active_num=-1, scale=None):
    """MoeInitRoutingV3, dropless (converter npu_moe_init_routing_v2.py:41-95; experiment_ops.h:2137-2192).
    Decisions: pairs are numbered f = t*K + k; gather index = sorted position -> f, scatter index = f -> position.
    active_expert_range [lo, hi): only those experts keep rows and are counted (expert_tokens has hi - lo entries);
    the other pairs sort behind the kept ones (stable), get no row, and -1 in the scatter index.  active_num > 0:
    only rows at sorted positions < active_num are materialised (the indices still describe the whole sort).
    scale: without quantisation a per-token fp32 value that is carried to the copies (expanded_scale); with dynamic
    quantisation fp32 smooth scales [hi - lo, H] or [1, H] multiplied in (fp32) before each copy is quantised on its own."""
    T, K = expert_idx.shape
    lo, hi = (0, expert_num) if active_expert_range is None else (int(active_expert_range[0]), int(active_expert_range[1]))
    nk = hi - lo
    flat = expert_idx.reshape(-1).to(torch.int64)
    keys = torch.where((flat >= lo) & (flat < hi), flat - lo, torch.full_like(flat, nk))
    order = torch.sort(keys, stable=True)
    kept = int((keys < nk).sum())
    tok = order.indices // K
    M, H = T * K, x.shape[1]
    limit = kept if active_num is None or active_num <= 0 else min(kept, int(active_num))
    if quant_mode == 1:
        if scale is None:
            q, s = dynamic_quant(x)
            ex_all, es_all = q[tok], s[tok]
        else:
            sm = scale.float().reshape(-1, H)
            srow = sm[order.values.clamp(max=nk - 1)] if sm.shape[0] > 1 else sm[:1].expand(M, H)
            ex_all, es_all = quantize_rows_f32(x[tok].float() * srow)
        ex = torch.zeros(M, H, dtype=torch.int8)
    else:
        ex_all = x[tok]
        es_all = scale.float()[tok] if scale is not None else torch.zeros(M, dtype=torch.float32)
        ex = torch.zeros(M, H, dtype=x.dtype)
    es = torch.zeros(M, dtype=torch.float32)
    ex[:limit] = ex_all[:limit]
    es[:limit] = es_all[:limit]
    if row_idx_type == 0:
        ridx = order.indices.to(torch.int32)
    else:
        ridx = torch.full((M,), -1, dtype=torch.int32)
        ridx[order.indices[:kept]] = torch.arange(kept, dtype=torch.int32)
    cnt = torch.bincount(keys, minlength=nk + 1)[:nk]
    tokens = cnt if expert_tokens_num_type == 1 else torch.cumsum(cnt, 0)
    return ex.contiguous(), ridx, tokens.to(torch.int64), es.contiguous()


# --------------------------------------------------------------------------------------------------
# npu_moe_distribute_dispatch / combine: R ranks simulated in one process
# --------------------------------------------------------------------------------------------------
@dataclass
class DispatchOut:
    expand_x: torch.Tensor          # [A, H] int8 (quant_mode 2) or input dtype (quant_mode 0)
    dynamic_scales: torch.Tensor    # [A] fp32
    expand_idx: torch.Tensor        # [T*K] int32: position of pair t*K+k in this rank's send order
    expert_token_nums: torch.Tensor  # [E_l] int64 counts (type 1) or cumsum (type 0)
    ep_recv_count: torch.Tensor     # [E_l*R] int32: rows for local expert e from source rank s at [e*R+s]
    tp_recv_count: torch.Tensor     # [1] int32, zero
    expand_scales: torch.Tensor     # [A] fp32, zero


def dispatch_rows(T: int, R: int, E: int, K: int) -> int:
    """Static worst-case row count of expand_x when global_bs == 0 (decision): T*R*min(E/R, K)."""
    return T * R * min(E // R, K)


def moe_distribute_dispatch(xs: Sequence[torch.Tensor], ids: Sequence[torch.Tensor], E: int,
                            quant_mode: int = 2, expert_token_nums_type: int = 1,
                            x_active_mask: Optional[Sequence[Optional[torch.Tensor]]] = None,
                            scales: Optional[torch.Tensor] = None, special_experts: int = 0,
                            global_bs: int = 0) -> List[DispatchOut]:
    """MoeDistributeDispatch for all R ranks at once (converter moe_distribute_dispatch.py:4-45).

    Rank r owns experts [r*E_l, (r+1)*E_l).  Each rank quantises its tokens once (quant_mode 2), sorts
    its T*K copies by expert id (stable in t*K+k) and sends each copy to the owner of its expert.  The
    receiver orders rows by (local expert, source rank, send order).  Decisions: the contents of the
    handshake tensors (see DispatchOut) and zero fill of rows past the received total.
    Optional arguments (decisions; the converters name them without defining them): x_active_mask[r] bool [T] --
    tokens marked False send nothing (their expand_idx entries are -1); scales fp32 [E, H] -- smooth scales: copy
    (t, k) is quantised on its own after the fp32 product x[t] * scales[expert]; special_experts > 0 (second-generation
    op, moe_distribute_dispatch_v2.py:15-18): ids in [E, E + special_experts) name zero / copy / constant experts
    that the combine evaluates at the sender, so those pairs are not sent either; global_bs != 0: the ranks may hold
    different numbers of tokens, at most global_bs / R each, and expand_x is sized for that maximum.
    """
    R = len(xs)
    E_l = E // R
    K = ids[0].shape[1]
    H = xs[0].shape[1]
    A = dispatch_rows(global_bs // R if global_bs else ids[0].shape[0], R, E, K)
    send_rows, send_scales, send_e, expand_idx = [], [], [], []
    for r in range(R):
        T = ids[r].shape[0]
        flat_e = ids[r].reshape(-1).to(torch.int64)
        keep = flat_e < E if special_experts > 0 else torch.ones_like(flat_e, dtype=torch.bool)
        if x_active_mask is not None and x_active_mask[r] is not None:
            keep = keep & x_active_mask[r].to(torch.bool).repeat_interleave(K)
        keys = torch.where(keep, flat_e, torch.full_like(flat_e, E))
        order = torch.sort(keys, stable=True)
        kept = int(keep.sum())
        tok = (order.indices // K)[:kept]
        if quant_mode == 2 and scales is not None:
            q, s = quantize_rows_f32(xs[r][tok].float() * scales.float()[order.values[:kept]])
        elif quant_mode == 2:
            q0, s0 = dynamic_quant(xs[r])
            q, s = q0[tok], s0[tok]
        elif quant_mode == 0:
            q, s = xs[r][tok], torch.zeros(kept, dtype=torch.float32)
        else:
            raise NotImplementedError("quant_mode must be 0 or 2")
        send_rows.append(q)
        send_scales.append(s)
        send_e.append(order.values[:kept])
        inv = torch.full((T * K,), -1, dtype=torch.int32)
        inv[order.indices[:kept]] = torch.arange(kept, dtype=torch.int32)
        expand_idx.append(inv)
    outs = []
    for d in range(R):
        rows, scales = [], []
        cnt = torch.zeros(E_l, R, dtype=torch.int32)
        for e in range(E_l):
            for s in range(R):
                sel = send_e[s] == d * E_l + e
                rows.append(send_rows[s][sel])
                scales.append(send_scales[s][sel])
                cnt[e, s] = int(sel.sum())
        rows = torch.cat(rows)
        scales = torch.cat(scales)
        ex = torch.zeros(A, H, dtype=rows.dtype)
        ds = torch.zeros(A, dtype=torch.float32)
        ex[:rows.shape[0]] = rows
        ds[:rows.shape[0]] = scales
        per_e = cnt.sum(dim=1).to(torch.int64)
        nums = per_e if expert_token_nums_type == 1 else torch.cumsum(per_e, 0)
        outs.append(DispatchOut(ex, ds, expand_idx[d], nums, cnt.reshape(-1).contiguous(),
                                torch.zeros(1, dtype=torch.int32), torch.zeros(A, dtype=torch.float32)))
    return outs


def special_expert_row(kind_index: int, ori_x: torch.Tensor, zero_num: int, copy_num: int, alpha_1=None, alpha_2=None,
                       const_v=None) -> torch.Tensor:
    """fp32 rows [T, H] that special expert number `kind_index` (its id minus moe_expert_num) stands for.  Decision (the
    second-generation combine names these inputs without defining them, moe_distribute_combine_v2.py:17-20,47-50): zero
    experts give 0, copy experts the token itself (ori_x), constant expert c gives alpha_1[c] * ori_x + alpha_2[c] *
    const_v[c], two fp32 products and one fp32 sum per element."""
    x = ori_x.float()
    if kind_index < zero_num:
        return torch.zeros_like(x)
    if kind_index < zero_num + copy_num:
        return x
    c = kind_index - zero_num - copy_num
    return alpha_1[c].float().unsqueeze(0) * x + alpha_2[c].float().unsqueeze(0) * const_v[c].float().unsqueeze(0)


def combine_rows(recv: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, E: int,
                 shared=None, x_active_mask=None, special=None) -> torch.Tensor:
    """weighted_gather_sum with the optional inputs: pairs of special experts (id >= E) take special_expert_row instead
    of a returned row; tokens whose mask is False give an all-zero output row (decision)."""
    T, K = weights.shape
    H = recv.shape[1] if recv.numel() else special["ori_x"].shape[1]
    acc = None
    for k in range(K):
        idk = ids[:, k].long()
        row = torch.zeros(T, H, dtype=torch.float32)
        normal = idk < E
        if special is None:
            normal = torch.ones_like(normal)
        p = pos[:, k].long()
        ok = normal & (p >= 0)
        row[ok] = recv[p[ok]].float()
        if special is not None:
            for sidx in torch.unique(idk[~normal]).tolist():
                sel = idk == sidx
                row[sel] = special_expert_row(int(sidx) - E, special["ori_x"], special["zero"], special["copy"],
                                              special.get("alpha_1"), special.get("alpha_2"), special.get("const_v"))[sel]
        term = weights[:, k].float().unsqueeze(-1) * row
        acc = term if acc is None else acc + term
    if shared is not None:
        acc = acc + shared.float()
    if x_active_mask is not None:
        acc[~x_active_mask.to(torch.bool)] = 0
    dtype = recv.dtype if recv.numel() else special["ori_x"].dtype
    return acc.to(dtype)


def moe_distribute_combine(ys: Sequence[torch.Tensor], ids: Sequence[torch.Tensor],
                           disp: Sequence[DispatchOut], weights: Sequence[torch.Tensor], E: int,
                           shared: Optional[Sequence[torch.Tensor]] = None,
                           x_active_mask: Optional[Sequence[Optional[torch.Tensor]]] = None,
                           special: Optional[Sequence[dict]] = None) -> List[torch.Tensor]:
    """MoeDistributeCombine for all R ranks (converter moe_distribute_combine.py:4-60).

    Every expert-output row returns to the rank that sent it, landing at its position in that rank's send
    order; then out[t] = sum_k expert_scales[t,k] * row(t,k) as in weighted_gather_sum (combine_rows when a mask or
    special experts are given: special[s] = {"ori_x", "zero", "copy", "alpha_1", "alpha_2", "const_v"} of rank s).
    """
    R = len(ys)
    E_l = E // R
    K = ids[0].shape[1]
    H = ys[0].shape[1]
    back = [[None] * R for _ in range(R)]      # back[src][owner] -> list of row blocks in expert order
    for d in range(R):
        cnt = disp[d].ep_recv_count.reshape(E_l, R).long()
        off = 0
        blocks = [[] for _ in range(R)]
        for e in range(E_l):
            for s in range(R):
                c = int(cnt[e, s])
                blocks[s].append(ys[d][off:off + c])
                off += c
        for s in range(R):
            back[s][d] = torch.cat(blocks[s]) if blocks[s] else torch.zeros(0, H, dtype=ys[d].dtype)
    outs = []
    for s in range(R):
        recv = torch.cat([back[s][d] for d in range(R)])      # == send order (sorted by global expert id)
        T = ids[s].shape[0]
        pos = disp[s].expand_idx.reshape(T, K)
        if x_active_mask is None and special is None:
            outs.append(weighted_gather_sum(recv, pos, weights[s], None if shared is None else shared[s]))
        else:
            outs.append(combine_rows(recv, pos, weights[s], ids[s], E, None if shared is None else shared[s],
                                     None if x_active_mask is None else x_active_mask[s], None if special is None else special[s]))
    return outs


# --------------------------------------------------------------------------------------------------
# whole layer
# --------------------------------------------------------------------------------------------------
@dataclass
class MoeWeights:
    w1: torch.Tensor   # [E, H, 2I] int8 gate_up
    s1: torch.Tensor   # [E, 2I] fp32
    w2: torch.Tensor   # [E, I, H] int8 down
    s2: torch.Tensor   # [E, H] fp32


def expert_ffn(ex: torch.Tensor, xs: torch.Tensor, counts: torch.Tensor, w: MoeWeights,
               collect: Optional[dict] = None) -> torch.Tensor:
    """gate_up GEMM (int32) -> dequant+SwiGLU+requant -> down GEMM (bf16) on rows grouped by expert."""
    h32 = grouped_matmul_w8a8(ex, w.w1, None, None, counts, 1, output_dtype=3)
    hq, hs = dequant_swiglu_quant(h32, w.s1, xs, counts, activate_left=True, quant_mode=1)
    y = grouped_matmul_w8a8(hq, w.w2, w.s2, hs, counts, 1, output_dtype=15)
    if collect is not None:
        collect.update(h32=h32, hq=hq, hs=hs, y=y)
    return y


def moe_layer(xs: Sequence[torch.Tensor], ids: Sequence[torch.Tensor], weights: Sequence[torch.Tensor],
              w: MoeWeights, collect: Optional[list] = None) -> List[torch.Tensor]:
    """The expert-parallel layer over R simulated ranks (R = len(xs); R = 1 is the single-GPU layer).

    dispatch(quant) -> expert FFN on each owner's slice of the weights -> combine.
    """
    R = len(xs)
    E = w.w1.shape[0]
    E_l = E // R
    disp = moe_distribute_dispatch(xs, ids, E, quant_mode=2, expert_token_nums_type=1)
    ys = []
    for r in range(R):
        sl = slice(r * E_l, (r + 1) * E_l)
        wr = MoeWeights(w.w1[sl], w.s1[sl], w.w2[sl], w.s2[sl])
        c = {} if collect is not None else None
        ys.append(expert_ffn(disp[r].expand_x, disp[r].dynamic_scales, disp[r].expert_token_nums, wr, c))
        if collect is not None:
            c.update(disp=disp[r])
            collect.append(c)
    return moe_distribute_combine(ys, ids, disp, weights, E)


# --------------------------------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# --------------------------------------------------------------------------------------------------
@dataclass
class MoeConfig:
    name: str
    T: int      # tokens per rank
    H: int
    E: int
    K: int
    I: int
    zipf_s: float = 0.0


CONFIGS = {
    "cfg0": MoeConfig("cfg0", 64, 1024, 8, 2, 512),
    "cfg1": MoeConfig("cfg1", 256, 7168, 256, 8, 2048),
    "cfg2": MoeConfig("cfg2", 128, 7168, 256, 8, 2048),
    "cfg3": MoeConfig("cfg3", 8192, 7168, 256, 8, 2048, zipf_s=1.2),
    "cfg4": MoeConfig("cfg4", 4096, 4096, 128, 8, 1536),
}


def make_tokens(cfg: MoeConfig, seed: int = 0, rank: int = 0):
    """x bf16 ~ N(0,1) [T,H]; router logits fp32 ~ N(0,1) (+ Zipf bias when cfg.zipf_s > 0) -> ids, weights."""
    g = torch.Generator().manual_seed(seed * 1000 + rank)
    x = torch.randn(cfg.T, cfg.H, generator=g, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn(cfg.T, cfg.E, generator=g, dtype=torch.float32)
    if cfg.zipf_s > 0:
        gp = torch.Generator().manual_seed(seed)
        perm = torch.randperm(cfg.E, generator=gp)
        p = (torch.arange(cfg.E, dtype=torch.float64) + 1.0) ** (-cfg.zipf_s)
        p = p / p.sum()
        logits = logits + torch.log(p)[perm].float()
    ids, w = gating_topk(logits, cfg.K)
    return x, ids, w


def make_weights(cfg: MoeConfig, seed: int = 0, experts: Optional[range] = None) -> MoeWeights:
    """int8 weights uniform in [-127,127]; per-output-channel fp32 scales ~ U(1e-3, 1e-2)."""
    experts = range(cfg.E) if experts is None else experts
    w1, s1, w2, s2 = [], [], [], []
    for e in experts:
        g = torch.Generator().manual_seed(seed * 100003 + 7919 * e + 1)
        w1.append(torch.randint(-127, 128, (cfg.H, 2 * cfg.I), generator=g, dtype=torch.int8))
        w2.append(torch.randint(-127, 128, (cfg.I, cfg.H), generator=g, dtype=torch.int8))
        s1.append(torch.rand(2 * cfg.I, generator=g) * 9e-3 + 1e-3)
        s2.append(torch.rand(cfg.H, generator=g) * 9e-3 + 1e-3)
    return MoeWeights(torch.stack(w1), torch.stack(s1), torch.stack(w2), torch.stack(s2))
