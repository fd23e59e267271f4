"""``get_npu_backend``: a torch.compile backend that replays the AOT FX graph on CUDA and captures it.

The reference's graph-capture mode executes every FX node as ``target(*args, **kwargs)`` under device-graph
capture and replays the captured graph afterwards (python/torchair/_acl_concrete_graph/fx2acl_converter.py:442-459,
acl_graph.py:931-1024, 1192-1220, 1290-1359).  On B200 the same structure is: AOT-autograd -> FX GraphModule whose
call_function targets are torch.ops.npu.* -> eager replay, or (modes "reduce-overhead"/"npugraph_ex") one
torch.cuda.CUDAGraph per input-shape key with static input buffers.  Graphs that contain an expert-parallel
exchange with more than one rank are replayed eagerly, because exact-size all-to-all splits need one host read.

Entry points keep the reference signatures: ``get_npu_backend(*, compiler_config=None, custom_decompositions={})``
(python/torchair/npu_fx_compiler.py:890-909) and ``register_fx_node_ge_converter``
(python/torchair/_ge_concrete_graph/fx2ge_converter.py:401-414).
"""
from __future__ import annotations

import functools
import logging
from typing import Any, Callable, Dict, List, Optional

import torch

from .configs import CompilerConfig

# ---- logger with the reference's extra EVENT level (python/torchair/core/utils.py:78-130) ----
EVENT_LEVEL = 35
logging.addLevelName(EVENT_LEVEL, "EVENT")
logger = logging.getLogger("torchair")
if not logger.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(logging.Formatter("[%(levelname)s] TORCHAIR(%(process)d,%(processName)s):%(asctime)s.%(msecs)03d "
                                      "[%(filename)s:%(lineno)d] %(message)s", datefmt="%Y-%m-%d %H:%M:%S"))
    logger.addHandler(_h)
    logger.setLevel(logging.ERROR)
    logger.propagate = False

counters = {"compiled_graphs": 0, "captures": 0, "replays": 0, "eager_runs": 0, "fused_gate_up": 0, "fused_down_combine": 0}

_CONVERTERS: Dict[Any, Callable] = {}


def register_fx_node_ge_converter(aten_op):
    """Decorator kept for plug-ins written against the reference; records the function on ``op._ge_converter``.

    Nothing is lowered to a graph IR on B200 (ops run through the dispatcher), so the converter is never called.
    """
    def deco(fn):
        _CONVERTERS[aten_op] = fn
        try:
            aten_op._ge_converter = fn
        except Exception:  # some callables refuse attributes
            pass
        return fn
    return deco


def declare_supported(cases):
    """Decorator of the reference's converter test tables (_ge_concrete_graph/supported_declaration.py); kept inert."""
    def deco(fn):
        fn.supported_cases = cases
        return fn
    return deco


# ---- FX pass: int32 grouped matmul followed by dequant_swiglu_quant -> one fused gate_up launch ----
def fuse_gate_up(gm: torch.fx.GraphModule) -> int:
    """Rewrites  npu_grouped_matmul(int8, output_dtype=int32) -> getitem 0 -> npu_dequant_swiglu_quant(dynamic)
    into npu_grouped_matmul_swiglu_quant_v2-equivalent fused launch when the int32 tensor has no other user.

    The reference does the same kind of rewrite with inductor pattern passes (python/torchair/patterns/*.py).
    """
    from . import ops  # noqa: F401  (the operators must be registered before their overloads are looked up)
    import operator
    gmm_ops = (torch.ops.npu.npu_grouped_matmul.default, torch.ops.npu.npu_grouped_matmul.List)
    fused = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target is not torch.ops.npu.npu_dequant_swiglu_quant.default:
            continue
        src = node.args[0]
        if not (isinstance(src, torch.fx.Node) and src.op == "call_function" and src.target is operator.getitem and src.args[1] == 0):
            continue
        gmm = src.args[0]
        if not (isinstance(gmm, torch.fx.Node) and gmm.op == "call_function" and gmm.target in gmm_ops):
            continue
        if len(src.users) != 1 or len(gmm.users) != 1:
            continue
        gk, dk = gmm.kwargs, node.kwargs
        if gk.get("output_dtype") != 3 or dk.get("quant_mode", 0) != 1 or dk.get("weight_scale") is None \
                or dk.get("activation_scale") is None or dk.get("group_index") is None:
            continue
        if any(dk.get(k) is not None for k in ("bias", "quant_scale", "quant_offset")) or dk.get("swiglu_mode", 0) != 0:
            continue
        if any(gk.get(k) for k in ("bias", "offset", "antiquant_scale", "antiquant_offset")):
            continue
        if gk.get("group_list") is not dk.get("group_index") or gk.get("group_list_type", 0) != 1 \
                or not isinstance(gk.get("group_list"), torch.fx.Node):
            continue  # dequant_swiglu_quant reads per-group COUNTS; fuse only when the matmul uses the same tensor
        x_list, w_list = gmm.args[0], gmm.args[1]
        if len(x_list) != 1 or len(w_list) != 1:
            continue
        with gm.graph.inserting_before(node):
            new = gm.graph.call_function(_fused_gate_up_call, (x_list[0], w_list[0], dk["weight_scale"], dk["activation_scale"],
                                                              gk["group_list"], bool(dk.get("activate_left", False)),
                                                              gk.get("tuning_config")))
        node.replace_all_uses_with(new)
        gm.graph.erase_node(node)
        gm.graph.erase_node(src)
        gm.graph.erase_node(gmm)
        fused += 1
    if fused:
        gm.graph.lint()
        gm.recompile()
        counters["fused_gate_up"] += fused
    return fused


def _fused_gate_up_call(x, w, w_scale, x_scale, group_counts, activate_left, tuning_config=None):
    from . import ops
    return ops.fused_gate_up(x, w, w_scale.reshape(w.shape[0], -1) if w_scale.dim() > 1 else w_scale.expand(w.shape[0], -1),
                             x_scale.reshape(-1), group_counts, 1, activate_left, expected_rows=ops._expected_rows(tuning_config))


def fuse_down_combine(gm: torch.fx.GraphModule) -> int:
    """Rewrites  npu_grouped_matmul(int8, 16-bit output) -> getitem 0 -> npu_moe_distribute_combine(expand_x=that)  into one
    step when the group has more than one rank and moves rows over peer memory: the GEMM's epilogue then stores its rows
    into the senders' return buffers (ops.fused_down_combine) and the intermediate [rows, H] tensor disappears."""
    import operator
    from . import ep
    gmm_ops = (torch.ops.npu.npu_grouped_matmul.default, torch.ops.npu.npu_grouped_matmul.List)
    comb_ops = (torch.ops.npu.npu_moe_distribute_combine.default, torch.ops.npu.npu_moe_distribute_combine_v2.default)
    fused = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target not in comb_ops or len(node.args) < 9:
            continue
        src = node.args[0]
        if not (isinstance(src, torch.fx.Node) and src.op == "call_function" and src.target is operator.getitem and src.args[1] == 0):
            continue
        gmm = src.args[0]
        if not (isinstance(gmm, torch.fx.Node) and gmm.op == "call_function" and gmm.target in gmm_ops):
            continue
        if len(src.users) != 1 or len(gmm.users) != 1:
            continue
        group, R = node.args[5], node.args[6]
        if not (isinstance(group, str) and isinstance(R, int) and R > 1):
            continue
        try:
            if ep.transport_of(group, True) != "peer":
                continue
        except RuntimeError:
            continue
        gk, ck = gmm.kwargs, node.kwargs
        if any(v is not None and k != "shared_expert_x" and v not in (0, 1, "") for k, v in ck.items()):
            continue     # only the shared-expert rows may be passed besides the positional arguments
        if any(gk.get(k) for k in ("bias", "offset", "antiquant_scale", "antiquant_offset")) or gk.get("output_dtype") not in (5, 15):
            continue
        x_list, w_list, sc, pts = gmm.args[0], gmm.args[1], gk.get("scale"), gk.get("per_token_scale")
        if len(x_list) != 1 or len(w_list) != 1 or not sc or not pts or len(sc) != 1 or len(pts) != 1:
            continue
        if not isinstance(gk.get("group_list"), torch.fx.Node):
            continue
        val = x_list[0].meta.get("val") if isinstance(x_list[0], torch.fx.Node) else None
        if val is None or val.dtype != torch.int8:
            continue
        with gm.graph.inserting_before(node):
            new = gm.graph.call_function(_fused_down_combine_call, (
                x_list[0], w_list[0], sc[0], pts[0], gk["group_list"], int(gk.get("group_list_type", 0) or 0), node.args[1],
                node.args[2], node.args[3], node.args[4], group, R, node.args[7], node.args[8], ck.get("shared_expert_x"),
                gk["output_dtype"], gk.get("tuning_config")))
        node.replace_all_uses_with(new)
        gm.graph.erase_node(node)
        gm.graph.erase_node(src)
        gm.graph.erase_node(gmm)
        fused += 1
    if fused:
        gm.graph.lint()
        gm.recompile()
        counters["fused_down_combine"] += fused
    return fused


def _fused_down_combine_call(hq, w2, s2, hs, group_list, group_list_type, expert_ids, expand_idx, ep_send_counts, expert_scales,
                             group_ep, R, rank, E, shared, output_dtype, tuning_config=None):
    from . import ops
    return ops.fused_down_combine(hq, w2, s2, hs.reshape(-1), group_list, group_list_type, expert_ids, expand_idx, ep_send_counts,
                                  expert_scales, group_ep, R, rank, E, shared,
                                  torch.bfloat16 if output_dtype == 15 else torch.float16,
                                  expected_rows=ops._expected_rows(tuning_config))


def _has_multi_rank_exchange(gm: torch.fx.GraphModule) -> bool:
    """True when the graph holds a dispatch or combine (either generation of the operators) over more than one rank
    whose group moves rows with NCCL: exact-size all-to-all splits need one host read, which no capture allows."""
    npu = torch.ops.npu
    dispatch_ops = (npu.npu_moe_distribute_dispatch.default, npu.npu_moe_distribute_dispatch_v2.default)
    combine_ops = (npu.npu_moe_distribute_combine.default, npu.npu_moe_distribute_combine_v2.default)
    for n in gm.graph.nodes:
        if n.op != "call_function" or n.target not in dispatch_ops + combine_ops:
            continue
        # (x, expert_ids, group_ep, ep_world_size, ...) and (expand_x, expert_ids, idx, counts, scales, group_ep, ep_world_size, ...)
        gi, wi = (2, 3) if n.target in dispatch_ops else (5, 6)
        group = n.args[gi] if len(n.args) > gi else n.kwargs.get("group_ep")
        ws = n.args[wi] if len(n.args) > wi else n.kwargs.get("ep_world_size")
        if not isinstance(ws, int) or ws > 1:
            from . import ep
            if not (isinstance(group, str) and ep.transport_of(group, True) == "peer"):
                return True
    return False


def _is_static_input(t) -> bool:
    """Parameters and tensors whose address the tracer marked as stable (buffers of inlined modules,
    torch._dynamo.mark_static_address) keep their storage between calls: the reference treats them as static
    addresses of its captured graph too (python/torchair/_acl_concrete_graph/fx2acl_converter.py:421-423)."""
    return isinstance(t, torch.nn.Parameter) or getattr(t, "_dynamo_static_input_type", None) is not None \
        or getattr(t, "_torchair_is_parameter", False)


class _CompiledFxGraph:
    """Callable returned to AOT-autograd: eager FX replay, or CUDA-graph capture/replay keyed by input shapes."""

    def __init__(self, gm: torch.fx.GraphModule, config: CompilerConfig):
        from . import scope
        self.gm = gm
        # graphs with stream scopes are replayed node by node on CUDA streams; the others run their generated code
        self.run = scope.StreamedReplay(gm) if scope.uses_scopes(gm) else gm
        self.capture = config.mode.raw in ("reduce-overhead", "npugraph_ex") and not config.debug.run_eagerly.raw \
            and not _has_multi_rank_exchange(gm)
        self.clone_input = bool(config.debug.aclgraph.clone_input.raw)
        # Parameters and static-address tensors are used in place, never cloned or copied per replay, as in the reference
        # (python/torchair/_acl_concrete_graph/acl_graph.py:263-278).  Without experimental_config.frozen_parameter their
        # addresses (and here also their version counters) join the capture key, so a moved or updated weight is captured
        # afresh; with it they are taken as frozen and the key is the input shapes alone.
        self.frozen = bool(config.experimental_config.frozen_parameter.raw)
        self.limit = int(config.debug.aclgraph.static_capture_size_limit.raw)
        self.graphs: Dict[Any, Any] = {}
        self.eager_forever = False

    def __call__(self, *args):
        with torch.profiler.record_function("npu_fx_compiler inference"):
            if not self.capture or self.eager_forever or not all(isinstance(a, torch.Tensor) and a.is_cuda for a in args):
                counters["eager_runs"] += 1
                return self.run(*args)
            static = [_is_static_input(a) for a in args]
            key = tuple((tuple(a.shape), a.dtype, a.device.index) + ((a.data_ptr(), a._version) if st and not self.frozen else ())
                        for a, st in zip(args, static))
            entry = self.graphs.get(key)
            if entry is None:
                if len(self.graphs) >= self.limit:
                    # same policy as the reference when captures overflow: fall back to eager for good
                    # (python/torchair/_acl_concrete_graph/acl_graph.py:1001-1014)
                    logger.warning("capture count exceeded static_capture_size_limit=%d; running eagerly", self.limit)
                    self.eager_forever = True
                    return self.run(*args)
                entry = self._capture(key, args, static)
            graph, static_in, static_out = entry
            for dst, src, st in zip(static_in, args, static):
                if not st and dst.data_ptr() != src.data_ptr():
                    dst.copy_(src)
            graph.replay()
            counters["replays"] += 1
            return static_out

    def _capture(self, key, args, static):
        static_in = [a if st or not self.clone_input else a.clone() for a, st in zip(args, static)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):      # warm-up off the capture: fills the packed-weight cache, loads kernels
            for _ in range(2):
                self.run(*static_in)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.profiler.record_function("npu_fx_compiler capture"), torch.cuda.graph(graph):
            static_out = self.run(*static_in)
        counters["captures"] += 1
        self.graphs[key] = (graph, static_in, static_out)
        return self.graphs[key]


def _npu_backend(gm: torch.fx.GraphModule, example_inputs: List[torch.Tensor], *, config: CompilerConfig,
                 decompositions: Dict):
    from torch._functorch.aot_autograd import aot_module_simplified
    from . import ops  # noqa: F401  (registers torch.ops.npu.*)

    def fw_compiler(fx_gm: torch.fx.GraphModule, inputs):
        pre, post = config.post_grad_custom_pre_pass.raw, config.post_grad_custom_post_pass.raw
        if callable(pre):
            pre(fx_gm.graph)
        if config.experimental_config.pattern_fusion_pass.raw:
            fuse_gate_up(fx_gm)
            fuse_down_combine(fx_gm)
        if callable(post):
            post(fx_gm.graph)
        fx_gm.recompile()
        counters["compiled_graphs"] += 1
        ignored = config.ignored_settings()
        if ignored:
            logger.warning("options without effect on B200 were set and are ignored: %s", ignored)
        return _CompiledFxGraph(fx_gm, config)

    return aot_module_simplified(gm, example_inputs, fw_compiler=fw_compiler, decompositions=decompositions)


def get_compiler(compiler_config: Optional[CompilerConfig] = None):
    """Signature of python/torchair/npu_fx_compiler.py:912-921; returns the FX-level compiler callable."""
    config = compiler_config if compiler_config is not None else CompilerConfig()

    def compiler(fx_gm, inputs):
        if config.experimental_config.pattern_fusion_pass.raw:
            fuse_gate_up(fx_gm)
            fuse_down_combine(fx_gm)
        return _CompiledFxGraph(fx_gm, config)
    return compiler


def get_npu_backend(*, compiler_config: CompilerConfig = None, custom_decompositions: Dict = {}):
    """Returns a callable usable as ``torch.compile(backend=...)`` (python/torchair/npu_fx_compiler.py:890-909)."""
    if compiler_config is None:
        compiler_config = CompilerConfig()
    if not isinstance(compiler_config, CompilerConfig):
        raise TypeError("compiler_config must be a CompilerConfig")
    return functools.partial(_npu_backend, config=compiler_config, decompositions=dict(custom_decompositions))
