"""torchair_b200: the W8A8 expert-parallel MoE path of Ascend/torchair, rebuilt for NVIDIA B200 (sm_100a).

Public surface mirrors the part of ``torchair`` that the path needs (python/torchair/__init__.py:1-80):
``get_npu_backend``, ``get_compiler``, ``CompilerConfig``, ``register_fx_node_ge_converter``, ``logger``; plus
``register_ep_group`` (group_ep names -> process groups) and ``install_as_torchair`` (makes ``import torchair``
resolve to this package so that scripts written against the reference run unchanged).  Importing the package
registers the ``torch.ops.npu.*`` operators; their kernels live in libtorchair_b200.so and there is no fallback.
"""
from __future__ import annotations

import sys

from . import _lib
from .configs import CompilerConfig
from .backend import get_compiler, get_npu_backend, register_fx_node_ge_converter, declare_supported, logger
from .ep import register_ep_group, get_ep_group, watchdog_of
from .watchdog import EpGroupFailed, EpWatchdog
from . import ops
from . import scope
from .ops import clear_weight_cache, gmm_status, gmm_status_reset, routing_status, check_status

__all__ = ["get_npu_backend", "get_compiler", "CompilerConfig", "register_fx_node_ge_converter", "logger",
           "register_ep_group", "watchdog_of", "EpGroupFailed", "EpWatchdog", "install_as_torchair", "clear_weight_cache", "gmm_status", "gmm_status_reset", "routing_status",
           "check_status", "scope",
           "use_internal_format_weight", "patch_for_hcom", "dynamo_export", "register_replacement", "npu_format_cast_via_cpu"]


def use_internal_format_weight(model, release_original: bool = False) -> None:
    """The reference casts a model's weights to the vendor's internal layout ahead of the first run
    (python/torchair/experimental/inference.py:99-110).  Here the counterpart is the one-off relayout of every int8
    [E, K, N] expert weight (parameter or buffer on a GPU) into the K-major packed form the grouped GEMM reads, so that
    the first forward, or a CUDA-graph capture, does not pay for it.

    release_original=True also frees the [E, K, N] original: the parameter's data becomes an [E, K, N] VIEW (strides
    (N*K, 1, K)) of the packed buffer.  Element for element it is the same tensor, so every consumer still sees the
    operator's layout, the grouped GEMM recognises the view and uses the buffer underneath as it is, and the weights are
    held once instead of twice (11.3 GB instead of 22.5 GB for the 256-expert decode layer)."""
    import torch
    done = 0
    for t in list(model.parameters()) + list(model.buffers()):
        if t.is_cuda and t.dtype == torch.int8 and t.dim() == 3:
            packed = ops.packed_weight(t)
            if release_original and packed.data_ptr() != t.data_ptr():
                with torch.no_grad():
                    t.data = packed.permute(0, 2, 1)
            done += 1
    if release_original:
        ops.clear_weight_cache()        # the cached relayouts now ARE the weights; entries keyed by the old storages go
    logger.info("use_internal_format_weight: %d expert weight tensors packed%s", done,
                ", originals released" if release_original else "")


def patch_for_hcom() -> None:
    """Kept for scripts that call it (python/torchair/__init__.py:53-70 patches torch.distributed for old PyTorch versions
    on Ascend).  Nothing needs patching here: collectives of a compiled graph run through torch.distributed as they are."""
    logger.info("patch_for_hcom: nothing to patch on this backend")


def _outside_the_path(name):
    def stub(*args, **kwargs):
        raise NotImplementedError(f"torchair.{name} drives the Ascend graph compiler and is outside the W8A8 MoE path "
                                  "this package implements")
    stub.__name__ = name
    stub.__doc__ = f"``torchair.{name}`` of the reference's public API; not part of the W8A8 MoE path: raises NotImplementedError."
    return stub


dynamo_export = _outside_the_path("dynamo_export")
register_replacement = _outside_the_path("register_replacement")
npu_format_cast_via_cpu = _outside_the_path("npu_format_cast_via_cpu")


def install_as_torchair() -> None:
    """Registers this package under the name ``torchair`` (no-op if a real torchair is already imported)."""
    sys.modules.setdefault("torchair", sys.modules[__name__])
    sys.modules.setdefault("torchair.configs", sys.modules[__name__ + ".configs"])
    sys.modules.setdefault("torchair.configs.compiler_config", sys.modules[__name__ + ".configs"])
    sys.modules.setdefault("torchair.scope", sys.modules[__name__ + ".scope"])
