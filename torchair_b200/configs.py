"""CompilerConfig: the attribute tree of the reference's configuration object.

Mirrors python/torchair/configs/compiler_config.py:24-60 and the option classes of
python/torchair/configs/_option_base.py:10-254: unknown attributes raise (``_option_base.py:221-232``), leaves hold
a value with optional allowed choices.  Only ``mode``, ``debug.run_eagerly``, ``debug.aclgraph.clone_input``,
``debug.aclgraph.static_capture_size_limit`` and the two custom-pass hooks change behaviour on B200; the leaves
that steer the Ascend graph engine are accepted so that existing scripts keep working, and ignored.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Sequence


class OptionValue:
    """A leaf: default + optional list of allowed values; ``.value`` stringifies like the reference."""

    def __init__(self, default: Any = None, choices: Optional[Sequence[Any]] = None, honoured: bool = False):
        self.default = default
        self.choices = None if choices is None else list(choices)
        self.honoured = honoured
        self._value = default

    @property
    def value(self):
        v = self._value
        if v is None:
            return None
        if isinstance(v, bool):
            return "1" if v else "0"
        return v if callable(v) else str(v)

    @value.setter
    def value(self, v):
        if self.choices is not None and v not in self.choices:
            raise ValueError(f"Please set legal value, got {v!r}, allowed {self.choices}")
        self._value = v

    @property
    def raw(self):
        return self._value


class NpuBaseConfig:
    """A node of the tree: attributes are fixed at construction; assigning to a leaf sets its value."""

    def __init__(self):
        object.__setattr__(self, "_fixed_attrs", set())

    def _add(self, **nodes):
        for k, v in nodes.items():
            object.__setattr__(self, k, v)
            self._fixed_attrs.add(k)

    def __setattr__(self, key, value):
        if key not in self._fixed_attrs:
            raise ValueError(f"{type(self).__name__} has no option {key!r}; available: {sorted(self._fixed_attrs)}")
        cur = object.__getattribute__(self, key)
        if isinstance(cur, OptionValue):
            cur.value = value
        else:
            raise ValueError(f"{key!r} is a group of options, not an option")

    def as_dict(self, prefix: str = "") -> Dict[str, Any]:
        out = {}
        for k in sorted(self._fixed_attrs):
            v = object.__getattribute__(self, k)
            if isinstance(v, OptionValue):
                out[prefix + k] = v.raw
            else:
                out.update(v.as_dict(prefix + k + "."))
        return out


def _group(**leaves) -> NpuBaseConfig:
    g = NpuBaseConfig()
    g._add(**leaves)
    return g


def _O(default=None, choices=None, honoured=False) -> OptionValue:
    return OptionValue(default, choices, honoured)


class CompilerConfig(NpuBaseConfig):
    """``CompilerConfig()`` takes no arguments (python/torchair/configs/compiler_config.py:24-45)."""

    MODES = ("max-autotune", "reduce-overhead", "npugraph_ex")

    def __init__(self):
        super().__init__()
        aclgraph_dbg = _group(
            disable_reinplace_inplaceable_ops_pass=_O(False, [True, False]),
            disable_reinplace_input_mutated_ops_pass=_O(False, [True, False]),
            disable_mempool_reuse_in_same_fx=_O(False, [True, False]),
            enable_output_clone=_O(False, [True, False]),
            static_capture_size_limit=_O(64, honoured=True),
            clone_input=_O(True, [True, False], honoured=True),
            remove_cat_ops=_O(True, [True, False]))
        debug = _group(
            graph_dump=_group(type=_O(None, [None, "txt", "pbtxt", "py"]), path=_O(None)),
            data_dump=_group(type=_O(None, [None, "npy"]), filter=_O(None), path=_O(None)),
            fx_summary=_group(type=_O(None, [None, "csv"]), skip_compile=_O(True, [True, False])),
            run_eagerly=_O(False, [True, False], honoured=True),
            deadlock_check=_O(False, [True, False]),
            aclgraph=aclgraph_dbg)
        experimental = _group(
            cc_parallel_enable=_O(False, [True, False]), keep_inference_input_mutations=_O(True, [True, False]),
            memory_efficiency=_O(False, [True, False]), frozen_parameter=_O(False, [True, False]),
            static_model_ops_lower_limit=_O(None), jit_compile=_O("auto", ["auto"]), npu_fx_pass=_O(False, [True, False]),
            aot_config_enable_joint_graph=_O(False, [True, False]), aot_config_output_loss_index=_O(0),
            topology_sorting_strategy=_O("DFS", ["BFS", "DFS", "RDFS", "StableRDFS"]), enable_ref_data=_O(False, [True, False]),
            enable_view_optimize=_O(True, [True, False]), remove_noop_ops=_O(True, [True, False]),
            tiling_schedule_optimize=_O(False, [True, False]), pattern_fusion_pass=_O(True, [True, False], honoured=True),
            aclgraph=_group(_aclnn_static_shape_kernel=_O(False, [True, False]),
                            _aclnn_static_shape_kernel_build_dir=_O(None),
                            _super_kernel_optimize=_O(False, [True, False]),
                            _super_kernel_debug_options=_O(None)))
        self._add(
            mode=_O("max-autotune", self.MODES, honoured=True),
            post_grad_custom_pre_pass=_O(None, honoured=True),
            post_grad_custom_post_pass=_O(None, honoured=True),
            debug=debug,
            experimental_config=experimental,
            dump_config=_group(enable_dump=_O(False, [True, False]), dump_path=_O(None), dump_mode=_O("all", ["input", "output", "all"]),
                               quant_dumpable=_O(False, [True, False]), dump_step=_O(None), dump_layer=_O(None),
                               dump_data=_O("tensor", ["tensor", "stats"]), dump_config_path=_O(None), data_dump_stage=_O(None)),
            ge_config=_group(enable_single_stream=_O(False, [True, False]), oo_level=_O("O3", ["O1", "O3"]),
                             oo_constant_folding=_O(None, [None, True, False]), oo_dead_code_elimination=_O(None, [None, True, False]),
                             export_compile_stat=_O("2", ["0", "1", "2"]), aicore_num=_O(None), optimization_switch=_O(None)),
            fusion_config=_group(fusion_switch_file=_O(None)),
            export=_group(export_mode=_O(False, [True, False]), export_path_dir=_O(None), export_name=_O(None),
                          weight_name=_O(None), inputs_name=_O(None),
                          experimental=_group(enable_record_nn_module_stack=_O(False, [True, False]),
                                              auto_atc_config_generated=_O(False, [True, False]),
                                              enable_lite_export=_O(False, [True, False]))),
            aoe_config=_group(aoe_mode=_O(None, [None, "2"]), work_path=_O(None), aoe_config_file=_O(None)),
            inference_config=_group(dynamic_gears_merge_policy=_O("zip", ["zip", "product"])),
            aclgraph_config=_group(use_custom_pool=_O(None)))

    def ignored_settings(self) -> Dict[str, Any]:
        """Leaves changed from their defaults that have no effect on B200 (for one warning at compile time)."""
        out = {}

        def walk(node, prefix):
            for k in sorted(node._fixed_attrs):
                v = object.__getattribute__(node, k)
                if isinstance(v, OptionValue):
                    if not v.honoured and v.raw != v.default:
                        out[prefix + k] = v.raw
                else:
                    walk(v, prefix + k + ".")

        walk(self, "")
        return out
