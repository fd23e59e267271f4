"""tab_moe_init_routing_static: routing for callers that cannot allocate device memory.

Some hosts bind the C library without owning an allocator on the GPU: a plugin that lives inside another
framework's memory pool, or a serving loop that fixed all of its allocations at start-up.  They cannot create the
workspace that tab_moe_init_routing asks for, so this entry point keeps the sort's scratch in a fixed array inside
the library instead.  The test calls it through the C ABI and requires bit-identical results to the
workspace-taking entry point, on two calls in a row (the second smaller than the first, so that anything left in
the shared scratch by the first call would show).  This file is named to be collected last.
"""
import ctypes

import pytest
import torch

from torchair_b200 import _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _route(entry, x, row, ids, active, bound):
    T, K = ids.shape
    H = x.shape[1]
    dev = x.device
    ex = torch.full((min(T, active) * K, H), -1.0, dtype=x.dtype, device=dev)
    eri = torch.full((T * K,), -1, dtype=torch.int32, device=dev)
    eei = torch.full((T * K,), -1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    if entry == "workspace":
        nbytes = _lib.workspace_bytes("tab_moe_init_routing_workspace_bytes", T, K, bound)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _lib.call("tab_moe_init_routing", _p(x), 15, _p(row), _p(ids), T, K, H, active, bound, _p(ex), _p(eri), _p(eei),
                  _p(ws), nbytes, stream)
    else:
        _lib.call("tab_moe_init_routing_static", _p(x), 15, _p(row), _p(ids), T, K, H, active, bound, _p(ex), _p(eri),
                  _p(eei), stream)
    torch.cuda.synchronize(dev)
    return ex, eri, eei


@pytest.mark.gpu
def test_static_scratch_routing_equals_workspace_routing_twice_in_a_row():
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(41)
    for T, K, E, H in ((4096, 8, 512, 64), (300, 4, 64, 256)):      # first call fills the scratch, second is smaller
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
        ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(dev)
        row = torch.arange(T * K, dtype=torch.int32).view(K, T).t().contiguous().to(dev)
        want = _route("workspace", x, row, ids, T, E)
        got = _route("static", x, row, ids, T, E)
        for a, b in zip(want, got):
            assert torch.equal(a, b)
        assert sorted(got[1].tolist()) == list(range(T * K))


def test_static_scratch_routing_rejects_sizes_beyond_its_array(built_library):
    one = ctypes.c_void_p(256)      # never dereferenced: the size check comes first
    n = ctypes.c_void_p(None)
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        _lib.call("tab_moe_init_routing_static", one, 15, one, one, 8192, 8, 64, 8192, 256, one, one, one, n)
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        _lib.call("tab_moe_init_routing_static", one, 15, one, one, 16, 2, 64, 16, 1024, one, one, one, n)
    _lib.call("tab_moe_init_routing_static", n, 15, n, n, 0, 8, 64, 0, 256, n, n, n, n)     # empty input: nothing to do
