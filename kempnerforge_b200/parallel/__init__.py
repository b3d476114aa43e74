"""Parallelism: mesh set-up, flat parameter storage, sharded data parallel, TP/SP, EP, PP.

The package also answers to the reference's name for it (kempnerforge/distributed) and exports what that package
exports, so ``from kempnerforge_b200.distributed import apply_ac, clip_grad_norm_, init_distributed`` works."""

from kempnerforge_b200.parallel.engine import DataParallelEngine, clip_grad_norm_
from kempnerforge_b200.parallel.flat import FlatParamGroup, flatten_model
from kempnerforge_b200.parallel.setup import (
    destroy_distributed,
    get_dp_info,
    get_world_info,
    init_distributed,
    is_rank_zero,
    mesh_dim,
    mesh_shape,
)

_LAZY = {   # resolved on first use: these modules import the model package, which imports this one
    "parallel": ("apply_ac", "apply_fsdp2", "build_parallel_model", "default_mp_policy", "get_dp_mesh"),
    "pipeline_parallel": ("build_pipeline_schedule", "build_pipeline_stage", "build_stage_module",
                          "compute_layer_assignment", "get_pp_mesh", "get_pp_rank", "get_pp_size"),
    "tensor_parallel": ("apply_tensor_parallel", "get_tp_mesh"),
}


def __getattr__(name: str):
    import importlib

    for module, names in _LAZY.items():
        if name in names:
            value = getattr(importlib.import_module(f"{__name__}.{module}"), name)
            globals()[name] = value
            return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = [n for n in dir() if not n.startswith("_")] + [n for names in _LAZY.values() for n in names]
