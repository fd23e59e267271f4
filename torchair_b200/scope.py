"""``torchair.scope``: stream scopes and tensor waits, replayed on CUDA streams.

The reference marks FX nodes with scope attributes through two side-effecting operators, ``air.scope_enter`` and
``air.scope_exit`` (python/torchair/scope/_scope.py:10-71), and orders a node behind another stream's result with
``air.wait_tensor`` (python/torchair/scope/_wait_tensor.py:7-44); its graph engine then places the nodes of an
``npu_stream_switch`` scope on a second device stream (python/torchair/scope/__init__.py:22-27,
python/torchair/_utils/graph_utils.py:17-55).  The documented use is the overlap of the shared experts' GEMMs with
the routed experts' dispatch.

On B200 the same three operators exist.  Run eagerly they do nothing (``wait_tensor`` raises, as in the reference).
In a compiled graph ``StreamedReplay`` executes the FX nodes of a scope on a CUDA stream of that label: a node waits
on an event of every input produced on another stream, every stream is forked from and joined back into the calling
stream, so the replay is legal inside CUDA-graph capture and becomes parallel branches of the captured graph.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
from torch.fx.node import has_side_effect

_lib = torch.library.Library("air", "FRAGMENT")

if not hasattr(torch.ops.air, "scope_enter"):
    _lib.define("scope_enter(str[] keys, str[] values, bool need_execute=False) -> ()")
    _lib.define("scope_exit(bool need_execute=False) -> ()")
    _lib.define("wait_tensor(Tensor self, Tensor dependency) -> Tensor")

    def _enter(keys: List[str], values: List[str], need_execute: bool = False) -> None:
        return None

    def _exit(need_execute: bool = False) -> None:
        return None

    def _wait_meta(self: torch.Tensor, dependency: torch.Tensor) -> torch.Tensor:
        return torch.empty_like(self)

    def _wait_eager(self: torch.Tensor, dependency: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError(
            "torch.ops.air.wait_tensor kernel_impl is not implemented! npu_wait_tensor is not support in this mode.")

    for _key in ("Meta", "CPU", "CUDA", "BackendSelect"):
        _lib.impl("scope_enter", _enter, _key)
        _lib.impl("scope_exit", _exit, _key)
    _lib.impl("wait_tensor", _wait_meta, "Meta")
    _lib.impl("wait_tensor", _wait_eager, "CPU")
    _lib.impl("wait_tensor", _wait_eager, "CUDA")

has_side_effect(torch.ops.air.scope_enter.default)
has_side_effect(torch.ops.air.scope_exit.default)

STREAM_LABEL = "_user_stream_label"
STREAM_PRIORITY = "_user_stream_priority"


class _Scope:
    def __init__(self, attrs: List[Tuple[str, str]]):
        self.attrs = attrs

    def __enter__(self):
        keys, values = zip(*self.attrs)
        return torch.ops.air.scope_enter(list(keys), list(values))

    def __exit__(self, *args):
        return torch.ops.air.scope_exit()


def npu_stream_switch(stream_tag: str, stream_priority: int = 0, enable_inner_parallel: bool = True):
    """Nodes created inside run on the stream named ``stream_tag`` (python/torchair/scope/__init__.py:22-27)."""
    return _Scope([(STREAM_LABEL, stream_tag), (STREAM_PRIORITY, str(stream_priority)),
                   ("_enable_inner_parallel", str(enable_inner_parallel))])


def npu_wait_tensor(self: torch.Tensor, dependency: torch.Tensor) -> torch.Tensor:
    """Returns ``self``, usable only after ``dependency`` has been computed (python/torchair/scope/__init__.py:5-8)."""
    return torch.ops.air.wait_tensor(self, dependency)


# Scopes whose attributes steer the vendor's kernel scheduler; they are recorded in the graph and have no effect here.
def super_kernel(scope: Optional[str], options: str = ""):
    return _Scope([("_super_kernel_scope", scope or ""), ("_super_kernel_options", options)])


def limit_core_num(op_aicore_num: int, op_vectorcore_num: int):
    return _Scope([("_op_aicore_num", str(op_aicore_num)), ("_op_vectorcore_num", str(op_vectorcore_num))])


def op_never_timeout(enable: bool = True):
    if not isinstance(enable, bool):
        raise TypeError(f"op_never_timeout() argument 'enable' must be bool, but got {type(enable).__name__}.")
    return _Scope([("_op_exec_never_timeout", str(enable))])


def data_dump():
    return _Scope([("torchair_enable_data_dump", "True")])


# --------------------------------------------------------------------------------------------------
# graph side
# --------------------------------------------------------------------------------------------------
_ENTER, _EXIT, _WAIT = "air.scope_enter.default", "air.scope_exit.default", "air.wait_tensor.default"


def uses_scopes(gm: torch.fx.GraphModule) -> bool:
    return any(n.op == "call_function" and str(n.target) in (_ENTER, _EXIT, _WAIT) for n in gm.graph.nodes)


def stream_plan(gm: torch.fx.GraphModule) -> Tuple[Dict[torch.fx.Node, Optional[str]], Dict[str, int]]:
    """Stream label of every node (None = the calling stream) and the priority asked for each label.

    Scopes nest; a scope without a stream label inherits the enclosing stream.  Unpaired enter/exit operators raise
    the RuntimeError the reference raises for them (python/torchair/npu_fx_compiler.py:419-468).
    """
    labels: Dict[torch.fx.Node, Optional[str]] = {}
    priorities: Dict[str, int] = {}
    stack: List[Tuple[torch.fx.Node, Optional[str]]] = []
    current: Optional[str] = None
    for node in gm.graph.nodes:
        name = str(node.target) if node.op == "call_function" else ""
        if name == _ENTER:
            stack.append((node, current))
            keys = list(node.args[0]) if node.args else list(node.kwargs.get("keys", []))
            values = list(node.args[1]) if len(node.args) > 1 else list(node.kwargs.get("values", []))
            attrs = dict(zip(keys, values))
            if STREAM_LABEL in attrs:
                current = attrs[STREAM_LABEL]
                priorities.setdefault(current, int(attrs.get(STREAM_PRIORITY, "0") or 0))
            labels[node] = current
        elif name == _EXIT:
            if not stack:
                raise RuntimeError(f"When you call the torch.ops.air.scope_exit operator: {node.name}, you must first call the "
                                   "torch.ops.air.scope_enter operator, as they must be called in pairs.")
            labels[node] = current
            current = stack.pop()[1]
        else:
            labels[node] = current
    if stack:
        raise RuntimeError("After you call the torch.ops.air.scope_enter operator, there is no paired call to the "
                           f"torch.ops.air.scope_exit operator. The parameters for these torch.ops.air.scope_enter calls are:"
                           f"{[n.args for n, _ in stack]}.")
    return labels, priorities


class CudaStreams:
    """The stream operations StreamedReplay needs, on CUDA.  Tests substitute a recorder with the same methods."""

    def __init__(self):
        self.side_streams: Dict[Tuple[int, str], Any] = {}

    def device_of(self, args):
        dev = next((a.device for a in args if isinstance(a, torch.Tensor) and a.is_cuda), None)
        if dev is None:
            raise RuntimeError("stream scopes need CUDA inputs")
        return dev

    def main(self, device):
        return torch.cuda.current_stream(device)

    def side(self, device, label: str, priority: int):
        key = (device.index if device.index is not None else torch.cuda.current_device(), label)
        s = self.side_streams.get(key)
        if s is None:
            s = self.side_streams[key] = torch.cuda.Stream(device=key[0], priority=-1 if priority > 0 else 0)
        return s

    def record(self, stream):
        ev = torch.cuda.Event()
        ev.record(stream)
        return ev

    def wait(self, stream, event) -> None:
        stream.wait_event(event)

    def on(self, stream):
        return torch.cuda.stream(stream)

    def mark(self, tensor: torch.Tensor, stream) -> None:
        if tensor.is_cuda:
            tensor.record_stream(stream)     # the allocator must not reuse the block before `stream` is done with it


class StreamedReplay:
    """Runs an FX graph node by node, each node on the stream of its scope.

    A plan is computed once: the stream label per node, which values cross streams (an event is recorded after the
    producer, the consumer's stream waits on it and the tensor is marked as used on that stream for the allocator),
    and the last use of every value (dropped right after, as the generated code of a GraphModule does).
    """

    def __init__(self, gm: torch.fx.GraphModule, streams=None):
        self.gm = gm
        self.rt = streams if streams is not None else CudaStreams()
        self.labels, self.priorities = stream_plan(gm)
        self.nodes = list(gm.graph.nodes)
        self.needs_event = set()      # values with a consumer on another stream
        last_use: Dict[torch.fx.Node, torch.fx.Node] = {}
        for n in self.nodes:
            for a in n.all_input_nodes:
                last_use[a] = n
                if self.labels.get(a) != self.labels.get(n):
                    self.needs_event.add(a)
        self.frees: Dict[torch.fx.Node, List[torch.fx.Node]] = {}
        for a, n in last_use.items():
            if n.op != "output":
                self.frees.setdefault(n, []).append(a)

    def stream_labels(self) -> List[str]:
        return sorted({l for l in self.labels.values() if l is not None})

    def _mark(self, value, stream) -> None:
        if isinstance(value, torch.Tensor):
            self.rt.mark(value, stream)
        elif isinstance(value, (list, tuple)):
            for v in value:
                self._mark(v, stream)

    def __call__(self, *args):
        rt = self.rt
        device = rt.device_of(args)
        main = rt.main(device)
        fork = None
        used: Dict[str, Any] = {}
        env: Dict[torch.fx.Node, Any] = {}
        events: Dict[torch.fx.Node, Any] = {}
        waited = set()                # (consumer stream label, producer) pairs already ordered
        it = iter(args)

        def stream_of(label):
            nonlocal fork
            if label is None:
                return main
            s = used.get(label)
            if s is None:
                if fork is None:
                    fork = rt.record(main)
                s = used[label] = rt.side(device, label, self.priorities.get(label, 0))
                rt.wait(s, fork)       # fork: what the caller queued before this call is visible to the side stream
            return s

        result = None
        for n in self.nodes:
            label = self.labels.get(n)
            if n.op == "placeholder":
                env[n] = next(it)
            elif n.op == "get_attr":
                env[n] = _fetch_attr(self.gm, n.target)
            elif n.op == "output":
                for s in used.values():       # join: the caller's stream continues after every side stream
                    rt.wait(main, rt.record(s))
                result = torch.fx.node.map_arg(n.args[0], lambda a: env[a])
                for a in n.all_input_nodes:
                    if self.labels.get(a) is not None:
                        self._mark(env[a], main)
            else:
                name = str(n.target) if n.op == "call_function" else ""
                if name in (_ENTER, _EXIT):
                    continue
                s = stream_of(label)
                for a in n.all_input_nodes:
                    if a in events and self.labels.get(a) != label and (label, a) not in waited:
                        waited.add((label, a))
                        rt.wait(s, events[a])
                        self._mark(env[a], s)
                a_args = torch.fx.node.map_arg(n.args, lambda a: env[a])
                a_kwargs = torch.fx.node.map_arg(n.kwargs, lambda a: env[a])
                if name == _WAIT:
                    env[n] = a_args[0]        # the wait itself happened above, through the dependency's event
                else:
                    with rt.on(s):
                        if n.op == "call_function":
                            env[n] = n.target(*a_args, **a_kwargs)
                        elif n.op == "call_method":
                            env[n] = getattr(a_args[0], n.target)(*a_args[1:], **a_kwargs)
                        else:
                            env[n] = self.gm.get_submodule(n.target)(*a_args, **a_kwargs)
                if n in self.needs_event:
                    events[n] = rt.record(s)
            for a in self.frees.get(n, ()):
                env.pop(a, None)
        return result


def _fetch_attr(gm: torch.nn.Module, target: str):
    obj = gm
    for part in target.split("."):
        obj = getattr(obj, part)
    return obj
