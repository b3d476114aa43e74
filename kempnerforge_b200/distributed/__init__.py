"""``kempnerforge_b200.distributed`` mirrors the reference's package name (kempnerforge/distributed): the modules
of ``kempnerforge_b200.parallel`` under their reference names, plus ``utils`` (``clip_grad_norm_``, ``get_dp_info``)."""

import importlib
import sys
import types

from kempnerforge_b200.parallel.engine import clip_grad_norm_  # noqa: F401
from kempnerforge_b200.parallel.parallel import build_parallel_model  # noqa: F401
from kempnerforge_b200.parallel.setup import get_dp_info, get_world_info, init_distributed  # noqa: F401

for _name in ("setup", "parallel", "tensor_parallel", "expert_parallel", "pipeline_parallel"):
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"kempnerforge_b200.parallel.{_name}")
    globals()[_name] = sys.modules[f"{__name__}.{_name}"]

utils = types.ModuleType(f"{__name__}.utils")
utils.clip_grad_norm_ = clip_grad_norm_
utils.get_dp_info = get_dp_info
sys.modules[utils.__name__] = utils
