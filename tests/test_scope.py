"""Stream scopes (torchair.scope): tracing into FX graphs and the stream plan of the replay, on CPU with a recorder in
place of the CUDA streams.  The reference's own test of this surface is tests/st/torchair_scope_st.py."""
import contextlib

import pytest
import torch
from torch._functorch.aot_autograd import aot_module_simplified

import torchair_b200 as tb
from torchair_b200 import scope


class Recorder:
    """Stands in for scope.CudaStreams: streams are their labels, every operation is logged."""

    def __init__(self):
        self.log = []

    def device_of(self, args):
        return torch.device("cpu")

    def main(self, device):
        return "main"

    def side(self, device, label, priority):
        self.log.append(("side", label, priority))
        return label

    def record(self, stream):
        self.log.append(("record", stream))
        return ("event", stream, len(self.log))

    def wait(self, stream, event):
        self.log.append(("wait", stream, event[1]))

    @contextlib.contextmanager
    def on(self, stream):
        self.log.append(("run", stream))
        yield

    def mark(self, tensor, stream):
        self.log.append(("mark", stream))


def _compile(fn, recorder, graphs):
    def backend(gm, example_inputs):
        def fw(g, inputs):
            graphs.append(g)
            return scope.StreamedReplay(g, streams=recorder)
        return aot_module_simplified(gm, example_inputs, fw_compiler=fw)
    return torch.compile(fn, backend=backend, fullgraph=True)


def test_stream_switch_and_wait_tensor_trace_and_replay():
    def shared_and_routed(x, w):
        routed = x @ w
        with scope.npu_stream_switch("shared", 1):
            shared = torch.relu(x) @ w
            shared = shared * 2
        routed = scope.npu_wait_tensor(routed, shared)
        return routed + shared

    rec, graphs = Recorder(), []
    x, w = torch.randn(4, 4), torch.randn(4, 4)
    got = _compile(shared_and_routed, rec, graphs)(x, w)
    torch.testing.assert_close(got, x @ w + (torch.relu(x) @ w) * 2)
    (g,) = graphs
    targets = [str(n.target) for n in g.graph.nodes if n.op == "call_function"]
    assert targets.count("air.scope_enter.default") == 1 and targets.count("air.scope_exit.default") == 1
    assert "air.wait_tensor.default" in targets
    enter = next(n for n in g.graph.nodes if str(n.target) == "air.scope_enter.default")
    assert enter.args[0][0] == "_user_stream_label" and enter.args[1][:2] == ["shared", "1"]
    labels, priorities = scope.stream_plan(g)
    by_name = {n.name: l for n, l in labels.items()}
    assert by_name["mm"] is None and by_name["relu"] == "shared" and by_name["mm_1"] == "shared" and by_name["mul"] == "shared"
    assert by_name["wait_tensor"] is None and by_name["add"] is None and priorities == {"shared": 1}
    # the replay: mm on main; fork (record main, shared waits); three nodes on shared, one event after the last; main waits
    # on it for wait_tensor (which launches nothing); add on main; join before the output
    assert rec.log == [
        ("run", "main"),
        ("record", "main"), ("side", "shared", 1), ("wait", "shared", "main"),
        ("run", "shared"), ("run", "shared"), ("run", "shared"), ("record", "shared"),
        ("wait", "main", "shared"), ("mark", "main"),
        ("run", "main"),
        ("record", "shared"), ("wait", "main", "shared"),
    ]


def test_nested_scopes_inherit_and_restore_the_stream():
    def fn(x):
        with scope.npu_stream_switch("a"):
            y = x + 1
            with scope.limit_core_num(8, 16):          # no stream label: stays on "a"
                y = y * 2
            with scope.npu_stream_switch("b"):
                z = x - 1
            y = y + 3
        return y + z

    rec, graphs = Recorder(), []
    x = torch.randn(8)
    torch.testing.assert_close(_compile(fn, rec, graphs)(x), (x + 1) * 2 + 3 + (x - 1))
    labels, _ = scope.stream_plan(graphs[0])
    seq = [(n.name, l) for n, l in labels.items() if n.op == "call_function" and not str(n.target).startswith("air.")]
    assert [l for _, l in seq] == ["a", "a", "b", "a", None]
    replay = scope.StreamedReplay(graphs[0], streams=Recorder())
    assert replay.stream_labels() == ["a", "b"]
    # both side streams are forked from main and joined back
    assert [e for e in rec.log if e[0] == "wait" and e[1] in ("a", "b")] == [("wait", "a", "main"), ("wait", "b", "main")]
    assert rec.log[-4:] == [("record", "a"), ("wait", "main", "a"), ("record", "b"), ("wait", "main", "b")]


def test_unpaired_scope_operators_raise_like_the_reference():
    g = torch.fx.Graph()
    x = g.placeholder("x")
    g.call_function(torch.ops.air.scope_exit.default, ())
    g.output(x)
    with pytest.raises(RuntimeError, match="must be called in pairs"):
        scope.stream_plan(torch.fx.GraphModule(torch.nn.Module(), g))
    g = torch.fx.Graph()
    x = g.placeholder("x")
    g.call_function(torch.ops.air.scope_enter.default, (["_user_stream_label"], ["s"]))
    g.output(x)
    with pytest.raises(RuntimeError, match="no paired call"):
        scope.stream_plan(torch.fx.GraphModule(torch.nn.Module(), g))


def test_eager_behaviour_and_module_alias():
    with scope.npu_stream_switch("s"):                 # eager: the scope operators do nothing
        y = torch.ones(2) + 1
    assert torch.equal(y, torch.full((2,), 2.0))
    with pytest.raises(NotImplementedError, match="not support in this mode"):
        scope.npu_wait_tensor(y, y)
    with pytest.raises(TypeError):
        scope.op_never_timeout("yes")
    tb.install_as_torchair()
    import torchair
    if torchair is tb:
        import torchair.scope as ts
        assert ts.npu_stream_switch is scope.npu_stream_switch
    assert not scope.uses_scopes(torch.fx.symbolic_trace(torch.nn.ReLU()))


def test_two_parallel_streams_as_in_the_reference_scope_test():
    """Shape of tests/st/torchair_scope_st.py:82-141: two stream scopes with their own priorities around independent work;
    the wait's result may even be dropped by the caller (then it orders nothing, as an unused value orders nothing in the
    reference's graph either) and the graph must still build and run."""
    def model(in1, in2, in3, in4):
        add_result = torch.add(in1, in2)
        with scope.npu_stream_switch('1', 2):
            scope.npu_wait_tensor(in4, add_result)
            mm_result = torch.mm(in3, in4)
        mm1 = torch.mm(in3, in4)
        with scope.npu_stream_switch('2', 3, False):
            in4b = scope.npu_wait_tensor(in4, mm_result)
            add2 = torch.add(in3, in4b)
        return add_result, mm_result, mm1, add2

    rec, graphs = Recorder(), []
    a = [torch.randn(4, 4) for _ in range(4)]
    got = _compile(model, rec, graphs)(*a)
    want = (a[0] + a[1], a[2] @ a[3], a[2] @ a[3], a[2] + a[3])
    for g, w in zip(got, want):
        torch.testing.assert_close(g, w)
    labels, priorities = scope.stream_plan(graphs[0])
    by_target = {}
    for n, l in labels.items():
        if n.op == "call_function" and not str(n.target).startswith("air."):
            by_target.setdefault(str(n.target), []).append(l)
    assert by_target["aten.mm.default"] == ['1', None] and by_target["aten.add.Tensor"] == [None, '2']
    assert priorities == {'1': 2, '2': 3}
    # stream '2' consumes mm_result of stream '1' through the kept wait: it must wait on an event recorded on '1'
    assert ("wait", "2", "1") in rec.log
