"""Host logic of the torch.compile backend that needs no GPU: which graphs may be captured, and which inputs of a
captured graph are used in place (reference: python/torchair/_acl_concrete_graph/fx2acl_converter.py:419-427,
acl_graph.py:263-278)."""
import pytest
import torch

import torchair_b200
from torchair_b200 import backend


def _graph(build):
    g = torch.fx.Graph()
    out = build(g)
    g.output(out)
    return torch.fx.GraphModule(torch.nn.Module(), g)


@pytest.mark.parametrize("gen", ["v1", "v2"])
@pytest.mark.parametrize("transport,world,expect", [("nccl", 2, True), ("nccl", 1, False), ("peer", 2, False)])
def test_multi_rank_nccl_exchange_keeps_a_graph_out_of_capture(gen, transport, world, expect):
    npu = torch.ops.npu
    disp = npu.npu_moe_distribute_dispatch.default if gen == "v1" else npu.npu_moe_distribute_dispatch_v2.default
    comb = npu.npu_moe_distribute_combine.default if gen == "v1" else npu.npu_moe_distribute_combine_v2.default
    name = f"g_{gen}_{transport}_{world}"
    torchair_b200.register_ep_group(name, object(), transport=transport)

    def with_dispatch(g):
        x, ids = g.placeholder("x"), g.placeholder("ids")
        return g.call_function(disp, (x, ids, name, world, 0, 8), {"quant_mode": 2})

    def with_combine(g):
        a = [g.placeholder(n) for n in ("y", "ids", "idx", "cnt", "w")]
        return g.call_function(comb, (*a, name, world, 0, 8))

    assert backend._has_multi_rank_exchange(_graph(with_dispatch)) is expect
    assert backend._has_multi_rank_exchange(_graph(with_combine)) is expect


def test_graph_without_exchange_may_be_captured():
    gm = _graph(lambda g: g.call_function(torch.ops.npu.npu_swiglu.default, (g.placeholder("x"),)))
    assert backend._has_multi_rank_exchange(gm) is False


def test_parameters_and_marked_tensors_are_static_inputs():
    p = torch.nn.Parameter(torch.zeros(2))
    t = torch.zeros(2)
    assert backend._is_static_input(p) and not backend._is_static_input(t)
    marked = torch.zeros(2)
    torch._dynamo.mark_static_address(marked)
    assert backend._is_static_input(marked)
    tagged = torch.zeros(2)
    tagged._torchair_is_parameter = True
    assert backend._is_static_input(tagged)


def test_compiled_module_passes_its_buffers_and_parameters_as_static_inputs():
    """What the capture relies on: the tensors AOT-autograd hands to the compiled callable for a module's weights are
    recognisable as static (not cloned, not copied per replay)."""
    seen = []

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.ones(4, 4))
            self.register_buffer("b", torch.ones(4))

        def forward(self, x):
            return x @ self.w + self.b

    def be(gm, example_inputs):
        from torch._functorch.aot_autograd import aot_module_simplified

        def fw(g, inputs):
            def run(*args):
                seen.append([backend._is_static_input(a) for a in args])
                return g(*args)
            return run
        return aot_module_simplified(gm, example_inputs, fw_compiler=fw)

    m = torch.compile(M(), backend=be, fullgraph=True)
    with torch.no_grad():
        m(torch.ones(2, 4))
    assert seen and sum(seen[0]) == 2 and len(seen[0]) == 3
