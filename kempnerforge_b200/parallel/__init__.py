"""Parallelism: mesh set-up, flat parameter storage, sharded data parallel, TP/SP, EP, PP."""

from kempnerforge_b200.parallel.engine import DataParallelEngine, clip_grad_norm_
from kempnerforge_b200.parallel.flat import FlatParamGroup, flatten_model
from kempnerforge_b200.parallel.setup import (
    destroy_distributed,
    get_dp_info,
    get_world_info,
    init_distributed,
    mesh_dim,
    mesh_shape,
)

__all__ = [n for n in dir() if not n.startswith("_")]
