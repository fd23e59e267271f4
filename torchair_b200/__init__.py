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
from .ep import register_ep_group, get_ep_group
from . import ops
from . import scope
from .ops import clear_weight_cache, gmm_status

__all__ = ["get_npu_backend", "get_compiler", "CompilerConfig", "register_fx_node_ge_converter", "logger",
           "register_ep_group", "install_as_torchair", "clear_weight_cache", "gmm_status", "scope"]


def install_as_torchair() -> None:
    """Registers this package under the name ``torchair`` (no-op if a real torchair is already imported)."""
    sys.modules.setdefault("torchair", sys.modules[__name__])
    sys.modules.setdefault("torchair.configs", sys.modules[__name__ + ".configs"])
    sys.modules.setdefault("torchair.configs.compiler_config", sys.modules[__name__ + ".configs"])
    sys.modules.setdefault("torchair.scope", sys.modules[__name__ + ".scope"])
