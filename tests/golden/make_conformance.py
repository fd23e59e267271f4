"""Generates tests/golden/conformance.json from the reference's own converter files.

Run where the reference project is checked out (REFERENCE_ROOT points at it):
    python tests/golden/make_conformance.py
It imports the reference's pure-Python converter layer over a stand-in for its native module
``torchair.core._torchair`` (the native module needs the vendor SDK and cannot be built), after this
repository's ``torch.ops.npu.*`` schemas are defined, and records for every hot-path op the converter's
parameter list (names, order, defaults, which are keyword-only).  The committed JSON lets the conformance
test run where the reference is absent.
"""
import importlib
import inspect
import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("REFERENCE_ROOT", "")     # checkout of the reference project; nothing is assumed when unset

CONVERTER_FILES = {
    "npu_moe_init_routing": "moe_init_routing",
    "npu_dynamic_quant": "npu_dynamic_quant",
    "npu_swiglu": "npu_swiglu",
    "npu_dequant_swiglu_quant": "npu_dequant_swiglu_quant",
    "npu_grouped_matmul": "grouped_matmul",
    "npu_grouped_matmul_swiglu_quant_v2": "grouped_matmul_swiglu_quant_v2",
    "npu_moe_distribute_dispatch": "moe_distribute_dispatch",
    "npu_moe_distribute_combine": "moe_distribute_combine",
    "npu_moe_compute_expert_tokens": "npu_moe_compute_expert_tokens",
    "npu_moe_gating_top_k_softmax": "moe_gating_top_k_softmax",
    "npu_moe_finalize_routing": "npu_moe_finalize_routing",
    "npu_moe_init_routing_v2": "npu_moe_init_routing_v2",
    "npu_moe_gating_top_k": "npu_moe_gating_top_k",
    "npu_moe_distribute_dispatch_v2": "moe_distribute_dispatch_v2",
    "npu_moe_distribute_combine_v2": "moe_distribute_combine_v2",
    "npu_grouped_matmul_finalize_routing": "grouped_matmul_finalize_routing",
    "npu_moe_gating_top_k_softmax_v2": "npu_moe_gating_top_k_softmax_v2",
}


def install_fake_native():
    fake = types.ModuleType("torchair.core._torchair")

    class TorchNpuGraphBase:
        def __init__(self, *a, **k):
            pass

    class TorchDataType:
        pass

    for i, n in enumerate(["BOOL", "UINT8", "INT8", "INT16", "INT32", "INT64", "BF16", "FLOAT16", "FLOAT32", "FLOAT64",
                           "COMPLEX32", "COMPLEX64", "COMPLEX128"]):
        setattr(TorchDataType, n, i)
    fake.TorchNpuGraphBase = TorchNpuGraphBase
    fake.TorchDataType = TorchDataType
    for n in ["InitializeGraphEngine", "FinalizeGraphEngine", "SetDebugLogPath", "GetSocName", "CheckAclnnAvaliable", "export",
              "AclopStartDumpArgs", "AclopStopDumpArgs", "AclmdlSetDump", "InitDeviceStdoutChannel", "StupidRepeat",
              "as_torch_tensors"]:
        setattr(fake, n, lambda *a, **k: None)
    fake.check_cann_compat = lambda *a, **k: ""
    fake.get_registered_ir_def = lambda *a, **k: ("None", [], [], [])
    sys.modules["torchair.core._torchair"] = fake


def describe(fn):
    params = []
    for p in inspect.signature(fn).parameters.values():
        if p.name == "meta_outputs":
            continue
        d = None if p.default is inspect.Parameter.empty else p.default
        params.append({"name": p.name, "kw_only": p.kind == inspect.Parameter.KEYWORD_ONLY,
                       "has_default": p.default is not inspect.Parameter.empty,
                       "default": d if isinstance(d, (int, float, str, bool, type(None))) else repr(d)})
    return params


def collect():
    if not REF or not os.path.isdir(os.path.join(REF, "python", "torchair")):
        raise RuntimeError("set REFERENCE_ROOT to a checkout of the reference project")
    sys.path.insert(0, ROOT)
    import torch
    import torchair_b200  # noqa: F401  defines torch.ops.npu.* first
    sys.modules.pop("torchair", None)
    sys.path.insert(0, os.path.join(REF, "python"))
    install_fake_native()
    import torchair  # the reference's python package  # noqa: F401
    out = {}
    for op, fname in CONVERTER_FILES.items():
        mod = importlib.import_module(f"torchair._ge_concrete_graph.ge_converter.custom.{fname}")
        overload = getattr(torch.ops.npu, op).default
        conv = getattr(overload, "_ge_converter", None)
        if conv is None:
            raise RuntimeError(f"reference converter did not attach to torch.ops.npu.{op}")
        fn = conv
        while hasattr(fn, "__wrapped__"):
            fn = fn.__wrapped__
        for attr in ("_aten_converter", "_converter", "converter"):
            if hasattr(conv, attr):
                fn = getattr(conv, attr)
        if not inspect.isfunction(fn):
            cands = [v for v in vars(mod).values() if inspect.isfunction(v) and v.__module__ == mod.__name__
                     and ("conve" in v.__name__)]
            fn = cands[0]
        out[op] = {"converter_file": f"python/torchair/_ge_concrete_graph/ge_converter/custom/{fname}.py",
                   "function": fn.__name__, "params": describe(fn)}
    import torchair as ref_pkg
    out["_api"] = {
        "get_npu_backend": str(inspect.signature(ref_pkg.get_npu_backend)),
        "CompilerConfig_modes": ["max-autotune", "reduce-overhead", "npugraph_ex"],
    }
    return out


if __name__ == "__main__":
    data = collect()
    with open(os.path.join(HERE, "conformance.json"), "w") as f:
        json.dump(data, f, indent=1, sort_keys=True)
    print("wrote conformance.json with", sorted(data))
