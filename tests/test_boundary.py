"""CPU tests of the drop-in boundary: C-ABI exports, argument validation, op schemas, shape rules, config."""
import ctypes
import inspect
import json
import os
import re

import pytest
import torch

import torchair_b200
from torchair_b200 import _lib, ops
from torchair_b200.backend import fuse_gate_up, counters

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "tab_api.h")).read()
    return sorted(set(re.findall(r"TAB_API\s+[\w\s\*]+?\b(tab_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_library):
    syms = _header_symbols()
    assert len(syms) >= 27
    for s in syms:
        assert hasattr(built_library, s), f"{s} is declared in include/tab_api.h but not exported"
    assert sorted(_lib.SIGNATURES) == syms, "python binding table and header disagree"
    assert built_library.tab_version() >= 100


def test_argument_validation_happens_before_any_cuda_call(built_library):
    n = ctypes.c_void_p(None)
    one = ctypes.c_void_p(16)   # fake aligned non-null address; validation must reject before it is touched
    cases = [
        ("tab_dynamic_quant", (one, 15, n, 4, 0, one, one, n), "rows"),
        ("tab_dynamic_quant", (one, 15, n, 4, 24, one, one, n), "multiple of 16"),
        ("tab_dynamic_quant", (one, 1, n, 4, 32, one, one, n), "dtype"),
        ("tab_dynamic_quant", (n, 15, n, 4, 32, one, one, n), "null"),
        ("tab_swiglu", (one, 15, 4, 31, one, n), "even"),
        ("tab_dequant_swiglu_quant", (one, one, 4, n, n, 0, 1, 8, 64, one, one, n), "group_index"),
        ("tab_moe_combine", (one, 3, one, one, n, 4, 2, 64, one, n), "dtype"),
        ("tab_moe_exchange_rows", (one, n, one, 2, 4, 0, 0, 24, 8, 1, one, n, n), "multiple of 16"),
        ("tab_moe_exchange_plan", (one, 64, 64, 0, 1, one, one, one, n), "R*E_l"),
        ("tab_grouped_matmul_w8a8", (one, one, n, n, n, one, 0, 8, 24, 64, 2, 15, one, 0, n), "Kd"),
        ("tab_grouped_matmul_w8a8", (one, one, n, n, n, one, 0, 8, 32, 64, 2000, 15, one, 0, n), "groups"),
        ("tab_grouped_matmul_w8a8", (one, one, n, n, n, one, 0, 8, 32, 64, 2, 1, one, 0, n), "output dtype"),
        ("tab_prepack_weight_i8", (one, 1, 32, 32, one, n), "in-place"),
    ]
    for name, args, needle in cases:
        with pytest.raises(RuntimeError) as ei:
            _lib.call(name, *args)
        assert needle in str(ei.value), (name, str(ei.value))
    with pytest.raises(RuntimeError):
        _lib.workspace_bytes("tab_moe_dispatch_pack_workspace_bytes", 4, 2, 100000)
    assert _lib.workspace_bytes("tab_grouped_matmul_swiglu_quant_workspace_bytes", 128, 512) >= 128 * 512 * 4 + 128 * 4


def test_zero_sized_calls_are_no_ops(built_library):
    n = ctypes.c_void_p(None)
    _lib.call("tab_dynamic_quant", n, 15, n, 0, 1024, n, n, n)
    _lib.call("tab_swiglu", n, 15, 0, 1024, n, n)
    _lib.call("tab_moe_combine", n, 15, n, n, n, 0, 8, 1024, n, n)
    _lib.call("tab_grouped_matmul_w8a8", n, n, n, n, n, n, 1, 0, 1024, 1024, 8, 15, n, 0, n)


def test_ops_have_no_cpu_fallback():
    x = torch.randn(4, 64)
    with pytest.raises(NotImplementedError):
        torch.ops.npu.npu_swiglu(x)
    with pytest.raises(NotImplementedError):
        torch.ops.npu.npu_dynamic_quant(x.to(torch.bfloat16))
    with pytest.raises(NotImplementedError):
        torch.ops.npu.npu_moe_init_routing(x, torch.zeros(4, 2, dtype=torch.int32), torch.zeros(4, 2, dtype=torch.int32), 4)
    with pytest.raises(NotImplementedError):
        torch.ops.npu.npu_dynamic_quant_asymmetric(x)


def test_meta_shape_rules():
    m = "meta"
    npu = torch.ops.npu
    x = torch.empty(6, 64, dtype=torch.bfloat16, device=m)
    ids = torch.empty(6, 2, dtype=torch.int32, device=m)
    ex, eri, eei = npu.npu_moe_init_routing(x, ids, ids, 4)
    assert ex.shape == (8, 64) and eri.shape == (12,) and eei.shape == (12,) and eri.dtype == torch.int32
    q, s = npu.npu_dynamic_quant(torch.empty(2, 3, 64, dtype=torch.float16, device=m))
    assert q.shape == (2, 3, 64) and q.dtype == torch.int8 and s.shape == (2, 3) and s.dtype == torch.float32
    assert npu.npu_swiglu(torch.empty(5, 64, device=m)).shape == (5, 32)
    assert npu.npu_swiglu(torch.empty(8, 5, device=m), 0).shape == (4, 5)
    y, sc = npu.npu_dequant_swiglu_quant(torch.empty(7, 128, dtype=torch.int32, device=m), quant_mode=1)
    assert y.shape == (7, 64) and y.dtype == torch.int8 and sc.shape == (7,)
    # error rules of python/torchair/_contrib/custom_torch_ops/auto_register_custom_torch_ops.py:121-156
    with pytest.raises(RuntimeError, match="larger than 1"):
        npu.npu_dequant_swiglu_quant(torch.empty(8, dtype=torch.int32, device=m))
    with pytest.raises(RuntimeError, match="even"):
        npu.npu_dequant_swiglu_quant(torch.empty(2, 7, dtype=torch.int32, device=m))
    with pytest.raises(RuntimeError, match="quant_mode"):
        npu.npu_dequant_swiglu_quant(torch.empty(2, 8, dtype=torch.int32, device=m), quant_mode=3)
    xq = torch.empty(16, 64, dtype=torch.int8, device=m)
    w = torch.empty(4, 64, 96, dtype=torch.int8, device=m)
    gl = torch.empty(4, dtype=torch.int64, device=m)
    for od, dt in ((3, torch.int32), (5, torch.float16), (15, torch.bfloat16)):
        out = npu.npu_grouped_matmul([xq], [w], group_list=gl, split_item=2, group_type=0, output_dtype=od)
        assert len(out) == 1 and out[0].shape == (16, 96) and out[0].dtype == dt
    with pytest.raises(ValueError):   # the reference rejects int8 output (grouped_matmul.py:188-194)
        npu.npu_grouped_matmul([xq], [w], group_list=gl, split_item=2, group_type=0, output_dtype=1)
    # output_bs == 0 means one output row per row of x (grouped_matmul_finalize_routing.py:113-114); only fp32 output
    fr = npu.npu_grouped_matmul_finalize_routing(xq, w, gl)
    assert fr.shape == (16, 96) and fr.dtype == torch.float32
    assert npu.npu_grouped_matmul_finalize_routing(xq, w, gl, output_bs=5, dtype=torch.float32).shape == (5, 96)
    with pytest.raises(RuntimeError, match="Not supported output dtype"):
        npu.npu_grouped_matmul_finalize_routing(xq, w, gl, dtype=torch.bfloat16)
    lg = torch.empty(5, 16, dtype=torch.bfloat16, device=m)
    yv, ev, sv = npu.npu_moe_gating_top_k_softmax_v2(lg, k=4, output_softmax=True)
    assert yv.shape == (5, 4) and yv.dtype == torch.bfloat16 and ev.dtype == torch.int32 and sv.shape == (5, 16) and sv.dtype == torch.float32
    assert npu.npu_moe_gating_top_k_softmax_v2(lg, k=4, renorm=1, output_softmax=True)[2].numel() == 0
    with pytest.raises(NotImplementedError):
        npu.npu_grouped_matmul([xq.to(torch.bfloat16)], [w], group_list=gl, split_item=2, group_type=0, output_dtype=15)
    hq, hs = npu.npu_grouped_matmul_swiglu_quant_v2(xq, [w], [torch.empty(4, 96, device=m)], torch.empty(16, device=m), gl)
    assert hq.shape == (16, 48) and hs.shape == (16,)
    R, E, T, K = 4, 16, 6, 2
    outs = npu.npu_moe_distribute_dispatch(x, ids, "ep", R, 1, E, quant_mode=2)
    A = T * R * min(E // R, K)
    assert [tuple(o.shape) for o in outs] == [(A, 64), (A,), (T * K,), (E // R,), (E,), (1,), (A,)]
    assert [o.dtype for o in outs] == [torch.int8, torch.float32, torch.int32, torch.int64, torch.int32, torch.int32, torch.float32]
    assert npu.npu_moe_distribute_dispatch(x, ids, "ep", R, 1, E, quant_mode=0)[0].dtype == torch.bfloat16
    out = npu.npu_moe_distribute_combine(torch.empty(A, 64, dtype=torch.bfloat16, device=m), ids, outs[2], outs[4],
                                         torch.empty(6, 2, device=m), "ep", R, 1, E)
    assert out.shape == (6, 64) and out.dtype == torch.bfloat16
    for bad in (dict(tp_world_size=2), dict(expert_shard_type=1), dict(shared_expert_rank_num=1), dict(quant_mode=1)):
        with pytest.raises(NotImplementedError):
            npu.npu_moe_distribute_dispatch(x, ids, "ep", R, 1, E, **bad)
    with pytest.raises(RuntimeError, match="global_bs"):          # must hold every rank's tokens: >= R * T, a multiple of R
        npu.npu_moe_distribute_dispatch(x, ids, "ep", R, 1, E, global_bs=8)
    big = npu.npu_moe_distribute_dispatch(x, ids, "ep", R, 1, E, quant_mode=2, global_bs=R * 10)
    assert big[0].shape == (10 * R * min(E // R, K), 64) and big[2].shape == (T * K,)
    with pytest.raises(RuntimeError):
        npu.npu_moe_distribute_dispatch(x, ids, "ep", 3, 1, E)     # E not divisible by R
    with pytest.raises(NotImplementedError):
        npu.npu_moe_distribute_combine(torch.empty(A, 64, dtype=torch.bfloat16, device=m), ids, outs[2], outs[4],
                                       torch.empty(6, 2, device=m), "ep", R, 1, E, comm_quant_mode=2)


def _schema_params(op_name):
    schema = getattr(torch.ops.npu, op_name).default._schema
    return [(a.name, a.kwarg_only, a.default_value if a.has_default_value() else inspect.Parameter.empty)
            for a in schema.arguments]


def test_schemas_match_the_reference_converters():
    """Names, order and keyword names are those of the reference's converter functions (committed snapshot)."""
    snap = json.load(open(os.path.join(ROOT, "tests", "golden", "conformance.json")))
    # converter-local names of positional arguments whose schema names (quoted in the converters' docstrings) differ
    renamed = {"input_data": "input", "skip2_optional": "skip2", "expert_for_source_row": "export_for_source_row"}
    for op, info in snap.items():
        if op.startswith("_"):
            continue
        ours = _schema_params(op)
        theirs = info["params"]
        assert [renamed.get(p["name"], p["name"]) for p in theirs] == [n for n, _, _ in ours], op
        for p, (name, kw_only, default) in zip(theirs, ours):
            if p["kw_only"]:
                assert kw_only, f"{op}.{name} must be keyword-only"
            if p["has_default"] and default is not inspect.Parameter.empty and p["default"] is not None \
                    and isinstance(p["default"], (int, float, str, bool)) and not (op == "npu_moe_init_routing"):
                if default is not None:
                    assert default == p["default"], f"{op}.{name}: default {default!r} != reference {p['default']!r}"
    assert snap["_api"]["CompilerConfig_modes"] == list(torchair_b200.CompilerConfig.MODES)


@pytest.mark.skipif(not os.environ.get("REFERENCE_ROOT") or
                    not os.path.isdir(os.path.join(os.environ["REFERENCE_ROOT"], "python", "torchair")),
                    reason="REFERENCE_ROOT does not point at a checkout of the reference")
def test_conformance_snapshot_is_fresh():
    import subprocess, sys
    code = ("import json,sys; sys.path.insert(0, %r); from tests.golden.make_conformance import collect; "
            "print('JSON'+json.dumps(collect(), sort_keys=True))" % ROOT)
    r = subprocess.run([sys.executable, "-W", "ignore", "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    live = json.loads([l for l in r.stdout.splitlines() if l.startswith("JSON")][-1][4:])
    snap = json.load(open(os.path.join(ROOT, "tests", "golden", "conformance.json")))
    assert live == snap


def test_public_api_signatures():
    sig = inspect.signature(torchair_b200.get_npu_backend)
    assert [(p.name, p.kind) for p in sig.parameters.values()] == \
        [("compiler_config", inspect.Parameter.KEYWORD_ONLY), ("custom_decompositions", inspect.Parameter.KEYWORD_ONLY)]
    assert sig.parameters["compiler_config"].default is None and sig.parameters["custom_decompositions"].default == {}
    assert callable(torchair_b200.get_npu_backend())
    with pytest.raises(TypeError):
        torchair_b200.get_npu_backend(compiler_config=object())
    assert torchair_b200.logger.name == "torchair"

    @torchair_b200.register_fx_node_ge_converter(torch.ops.npu.npu_swiglu.default)
    def conv(*a, **k):
        return None
    assert torch.ops.npu.npu_swiglu.default._ge_converter is conv
    torchair_b200.install_as_torchair()
    import torchair
    assert torchair.get_npu_backend is torchair_b200.get_npu_backend and torchair.CompilerConfig is torchair_b200.CompilerConfig


def test_compiler_config_tree():
    c = torchair_b200.CompilerConfig()
    assert c.mode.value == "max-autotune"
    c.mode = "reduce-overhead"
    assert c.mode.value == "reduce-overhead"
    with pytest.raises(ValueError):
        c.mode = "fastest"
    with pytest.raises(ValueError):
        c.not_an_option = 1
    with pytest.raises(ValueError):
        c.debug.aclgraph.no_such = 1
    with pytest.raises(ValueError):
        c.debug = 3
    c.debug.run_eagerly = True
    assert c.debug.run_eagerly.value == "1"
    c.debug.aclgraph.static_capture_size_limit = 4
    c.ge_config.oo_level = "O1"
    c.experimental_config.frozen_parameter = True
    assert c.ignored_settings() == {"ge_config.oo_level": "O1", "experimental_config.frozen_parameter": True}
    d = c.as_dict()
    assert d["mode"] == "reduce-overhead" and d["debug.aclgraph.static_capture_size_limit"] == 4


def test_fx_pass_fuses_int32_matmul_with_dequant_swiglu_quant():
    from torch.fx.experimental.proxy_tensor import make_fx
    npu = torch.ops.npu

    def unfused(x, w, s1, xs, counts):
        h32 = npu.npu_grouped_matmul([x], [w], group_list=counts, split_item=2, group_type=0, group_list_type=1, output_dtype=3)[0]
        return npu.npu_dequant_swiglu_quant(h32, weight_scale=s1, activation_scale=xs, group_index=counts,
                                            activate_left=True, quant_mode=1)

    m = "meta"
    args = (torch.empty(16, 64, dtype=torch.int8, device=m), torch.empty(4, 64, 96, dtype=torch.int8, device=m),
            torch.empty(4, 96, device=m), torch.empty(16, device=m), torch.empty(4, dtype=torch.int64, device=m))
    gm = make_fx(unfused)(*args)
    before = counters["fused_gate_up"]
    assert fuse_gate_up(gm) == 1 and counters["fused_gate_up"] == before + 1
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert torch.ops.npu.npu_grouped_matmul.default not in targets
    assert torch.ops.npu.npu_dequant_swiglu_quant.default not in targets

    def other_user(x, w, s1, xs, counts):       # the int32 tensor escapes: must stay unfused
        h32 = npu.npu_grouped_matmul([x], [w], group_list=counts, split_item=2, group_type=0, group_list_type=1, output_dtype=3)[0]
        q, s = npu.npu_dequant_swiglu_quant(h32, weight_scale=s1, activation_scale=xs, group_index=counts,
                                            activate_left=True, quant_mode=1)
        return q, s, h32
    assert fuse_gate_up(make_fx(other_user)(*args)) == 0


def test_fx_pass_fuses_down_matmul_with_combine_only_over_peer_memory():
    from torch.fx.experimental.proxy_tensor import make_fx
    from torchair_b200.backend import fuse_down_combine
    import torchair_b200
    npu = torch.ops.npu
    torchair_b200.register_ep_group("fx_peer", object(), transport="peer")
    torchair_b200.register_ep_group("fx_nccl", object(), transport="nccl")

    def make(group, world, keep_rows=False):
        def fn(hq, w2, s2, hs, counts, ids, expand_idx, ep_recv, wt):
            y = npu.npu_grouped_matmul([hq], [w2], scale=[s2], per_token_scale=[hs], group_list=counts, split_item=2, group_type=0,
                                       group_list_type=1, output_dtype=15)[0]
            out = npu.npu_moe_distribute_combine(y, ids, expand_idx, ep_recv, wt, group, world, 0, 8)
            return (out, y) if keep_rows else out
        return fn

    m = "meta"
    T, K, H, I, E_l, R = 8, 2, 64, 32, 4, 2
    A = T * R * min(E_l, K)
    args = (torch.empty(A, I, dtype=torch.int8, device=m), torch.empty(E_l, I, H, dtype=torch.int8, device=m),
            torch.empty(E_l, H, device=m), torch.empty(A, device=m), torch.empty(E_l, dtype=torch.int64, device=m),
            torch.empty(T, K, dtype=torch.int32, device=m), torch.empty(T * K, dtype=torch.int32, device=m),
            torch.empty(E_l * R, dtype=torch.int32, device=m), torch.empty(T, K, device=m))
    before = counters["fused_down_combine"]
    gm = make_fx(make("fx_peer", R))(*args)
    assert fuse_down_combine(gm) == 1 and counters["fused_down_combine"] == before + 1
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert npu.npu_grouped_matmul.default not in targets and npu.npu_moe_distribute_combine.default not in targets
    assert fuse_down_combine(make_fx(make("fx_nccl", R))(*args)) == 0          # NCCL transport: rows are sent by the collective
    assert fuse_down_combine(make_fx(make("fx_peer", 1))(*args[:5], *args[5:])) == 0   # one rank: nothing to send
    assert fuse_down_combine(make_fx(make("fx_peer", R, keep_rows=True))(*args)) == 0   # the rows escape: must stay


def test_remaining_public_names_of_the_reference_exist():
    """python/torchair/__init__.py:1-3 lists the package's public names.  Those beside the path either do their B200
    counterpart (use_internal_format_weight, patch_for_hcom) or say that they are outside it."""
    import torchair_b200 as tb
    for name in ("get_compiler", "get_npu_backend", "dynamo_export", "CompilerConfig", "use_internal_format_weight", "logger",
                 "register_fx_node_ge_converter", "patch_for_hcom", "register_replacement", "npu_format_cast_via_cpu"):
        assert hasattr(tb, name), name
    tb.patch_for_hcom()
    model = torch.nn.Linear(4, 4)
    model.register_buffer("experts", torch.zeros(2, 4, 4, dtype=torch.int8))
    assert tb.use_internal_format_weight(model) is None          # CPU tensors are left alone
    for fn in (tb.dynamo_export, tb.register_replacement, tb.npu_format_cast_via_cpu):
        with pytest.raises(NotImplementedError, match="outside the W8A8 MoE path"):
            fn(model)
