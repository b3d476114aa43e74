"""Applies the parallelism / precision / memory transformations to a model in the one order that works:

    tensor parallel -> expert parallel -> fp8 -> activation checkpointing -> sharded data parallel

TP must see whole weights before anything shards them, EP must slice experts before the flat buffers
are built, the fp8 conversion must happen before checkpointing wraps the block's forward, and the
data-parallel engine flattens whatever parameters are left on this rank.

Parity: kempnerforge/distributed/parallel.py:5-10,72-122,125-174,250-302,499-597 (same order, same
``apply_*`` entry points and ``build_parallel_model`` signature; mixed precision = parameters in
``param_dtype``; AC modes none / full / selective).
"""

from __future__ import annotations

from dataclasses import dataclass

import os

import logging

import torch
from torch import nn

from kempnerforge_b200.config.registry import registry
import kempnerforge_b200.models  # noqa: F401  (registers the built-in model builders)
from kempnerforge_b200.parallel.engine import DataParallelEngine
from kempnerforge_b200.parallel.setup import mesh_dim

log = logging.getLogger(__name__)


def get_dp_mesh(device_mesh):
    """The data-parallel sub-device_mesh: 1-D ``dp_shard`` or 2-D ``(dp_replicate, dp_shard)``; None if absent."""
    if device_mesh is None:
        return None
    names = device_mesh.mesh_dim_names or ()
    has_rep, has_shard = "dp_replicate" in names, "dp_shard" in names
    if has_rep and has_shard:
        return device_mesh["dp_replicate", "dp_shard"]
    if has_shard:
        return device_mesh["dp_shard"]
    if has_rep:
        return device_mesh["dp_replicate"]
    return None


def dp_process_group(mesh):
    """One process group spanning every data-parallel rank (replicate x shard), or None."""
    dp = get_dp_mesh(mesh)
    if dp is None:
        return None
    if dp.ndim == 1:
        return dp.get_group()
    return dp._flatten("dp").get_group() if hasattr(dp, "_flatten") else dp.get_group(0)


def apply_ac(model: nn.Module, mode: str = "full") -> None:
    """Activation checkpointing: ``full`` recomputes whole blocks, ``selective`` only attention."""
    mode = str(mode)
    if mode not in ("none", "full", "selective"):
        raise ValueError(f"Unknown activation_checkpointing mode: {mode!r}")
    n = 0
    for m in model.modules():
        if hasattr(m, "ac_mode"):
            m.ac_mode = mode
            n += 1
    log.info("activation checkpointing = %s on %d blocks", mode, n)


def apply_float8(model: nn.Module, enable_fsdp_float8_all_gather: bool = True) -> int:
    """Switch the dense Linear call sites to tensor-wise scaled fp8 GEMMs; experts, shared experts and routers
    keep bf16 (same module filter as the reference).  Returns the number of converted modules."""
    from kempnerforge_b200.ops import fp8

    return fp8.convert_model(model, skip=("experts", "shared_expert", "router"))


def _wants_sharded_params(model: nn.Module, world: int, mode: str | None) -> bool:
    """``resident``: every rank keeps whole parameters and gradients (fastest; 4 bytes per parameter per GPU);
    ``sharded``: ZeRO-3, 1/N of everything per rank; ``auto`` (default): sharded only when the resident plan would
    take more than half of the GPU's memory."""
    mode = (mode or os.environ.get("KF_DP_PARAM_SHARDING", "auto")).lower()
    if world <= 1 or mode == "resident":
        return False
    if mode == "sharded":
        return True
    if not torch.cuda.is_available():
        return False
    n = sum(p.numel() for p in model.parameters() if p.requires_grad)
    resident_bytes = 4 * n + 4 * n // world
    return resident_bytes > 0.5 * torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory


def _sharded_params_supported(model: nn.Module) -> str | None:
    """None when the model can train with sharded parameters, else the reason it cannot."""
    if getattr(model, "tp", None) is not None or getattr(model, "ep_group", None) is not None:
        return "tensor- or expert-parallel models keep the resident engine"
    layers = None
    for mod in model.modules():
        if isinstance(getattr(mod, "layers", None), nn.ModuleDict):
            layers = mod.layers
            break
    if layers is None:
        return "no block stack"
    for block in layers.values():
        if type(getattr(block, "mlp", None)).__name__ != "SwiGLUMLP" or getattr(block, "fp8", False):
            return "only dense bf16 SwiGLU blocks (the fused block path) are supported"
    return None


def apply_fsdp2(model: nn.Module, mesh, transport: str | None = None, reshard_after_forward: bool | None = None,
                param_sharding: str | None = None, **_) -> DataParallelEngine:
    """Flatten the model's parameters per block and shard optimizer state — and, in the ``sharded`` plan, parameters
    and gradients too (``reshard_after_forward`` semantics of kempnerforge/distributed/parallel.py:250-302) — over
    the data-parallel group."""
    pg = dp_process_group(mesh)
    allocator = None
    if transport is None:
        transport = os.environ.get("KF_DP_TRANSPORT", "auto")
    if transport == "auto":
        # our peer-memory kernels when the job is plain data parallelism on GPUs of one NVLink domain;
        # library collectives otherwise (other mesh dimensions, CPU, several nodes)
        # other mesh dimensions do not matter to the data-parallel transport (it lives on the dp sub-group); replicas of
        # a hybrid mesh are one flattened group.  KF_DP_SYMM_MIXED=0 restricts it to pure data parallelism.
        mixed_ok = os.environ.get("KF_DP_SYMM_MIXED", "1") != "0"
        pure_dp = mesh is not None and (mixed_ok or all(mesh_dim(mesh, d)[1] <= 1 for d in ("tp", "ep", "pp", "dp_replicate")))
        one_node = int(os.environ.get("LOCAL_WORLD_SIZE", "0") or 0) == int(os.environ.get("WORLD_SIZE", "1") or 1)
        on_gpu = torch.cuda.is_available() and pg is not None and "nccl" in str(torch.distributed.get_backend(pg))
        transport = "symmetric" if (pure_dp and one_node and on_gpu and torch.distributed.get_world_size(pg) > 1) else "collective"
    if transport == "symmetric":
        try:
            from kempnerforge_b200.comm import symmetric

            allocator = symmetric.make_allocator(pg)
            allocator(16, torch.bfloat16, torch.device("cuda", torch.cuda.current_device()))  # probe the rendezvous once
        except Exception as e:  # noqa: BLE001  symmetric memory is optional: fall back, loudly
            log.warning("symmetric-memory transport unavailable (%s); using library collectives", e)
            transport, allocator = "collective", None
    world = torch.distributed.get_world_size(pg) if pg is not None else 1
    if reshard_after_forward is False and param_sharding is None:
        param_sharding = "resident"
    if _wants_sharded_params(model, world, param_sharding):
        why = _sharded_params_supported(model)
        if why is None:
            from kempnerforge_b200.parallel.zero3 import ShardedDataParallelEngine

            if allocator is None and torch.cuda.is_available() and pg is not None and world > 1 \
                    and "nccl" in str(torch.distributed.get_backend(pg)) \
                    and int(os.environ.get("LOCAL_WORLD_SIZE", "0") or 0) == int(os.environ.get("WORLD_SIZE", "1") or 1) \
                    and os.environ.get("KF_DP_TRANSPORT", "auto") != "collective":
                # the sharded engine's kernels work on any mesh whose data-parallel group sits on one NVLink domain
                try:
                    from kempnerforge_b200.comm import symmetric

                    allocator = symmetric.make_allocator(pg)
                    allocator(16, torch.bfloat16, torch.device("cuda", torch.cuda.current_device()))
                except Exception as e:  # noqa: BLE001
                    log.warning("symmetric memory unavailable for the sharded engine (%s); using library collectives", e)
                    allocator = None
            log.info("data parallelism: sharded parameters (ZeRO-3) over %d ranks", world)
            return ShardedDataParallelEngine(model, pg, transport=transport, allocator=allocator)
        log.warning("sharded parameters requested but not available: %s", why)
    return DataParallelEngine(model, pg, transport=transport, allocator=allocator)


@dataclass(frozen=True)
class MixedPrecisionPolicy:
    """What the data-parallel engine does with dtypes: parameters and activations in ``param_dtype``, gradient
    reduction and optimizer state in ``reduce_dtype`` (fp32), module inputs cast to ``param_dtype``."""

    param_dtype: torch.dtype = torch.bfloat16
    reduce_dtype: torch.dtype = torch.float32
    cast_forward_inputs: bool = True


def default_mp_policy(param_dtype: torch.dtype = torch.bfloat16) -> MixedPrecisionPolicy:
    """Parity: kempnerforge/distributed/parallel.py:72-88."""
    return MixedPrecisionPolicy(param_dtype=param_dtype)


def build_parallel_model(
    model_config,
    device: torch.device,
    device_mesh=None,
    *,
    ac_mode: str = "none",
    param_dtype: torch.dtype = torch.bfloat16,
    fp8: bool = False,
    compile_model: bool = False,
    transport: str | None = None,
    vlm_config=None,
    ep_in_dp: bool = False,
    vision_config=None,
    adapter_config=None,
    mp_policy: MixedPrecisionPolicy | None = None,
    frames_per_clip: int = 1,
    param_sharding: str | None = None,
    **model_kwargs,
) -> nn.Module:
    """Build the registered model and apply TP -> EP -> FP8 -> AC -> sharded DP.

    ``mp_policy`` (see ``default_mp_policy``) overrides ``param_dtype``.  With ``vision_config`` and ``adapter_config``
    given as well as ``vlm_config`` the result is the vision-language wrapper of ``build_parallel_vlm``.
    """
    if mp_policy is not None:
        if mp_policy.reduce_dtype != torch.float32:
            raise ValueError("gradients are reduced in fp32; other reduce dtypes are not supported")
        param_dtype = mp_policy.param_dtype
    if vision_config is not None:
        if vlm_config is None or adapter_config is None:
            raise ValueError("a vision-language model needs vision_config, adapter_config and vlm_config together")
        from types import SimpleNamespace

        job = SimpleNamespace(model=model_config, vision_encoder=vision_config, adapter=adapter_config, vlm=vlm_config,
                              video=SimpleNamespace(max_frames=frames_per_clip) if frames_per_clip != 1 else None,
                              train=SimpleNamespace(param_dtype=param_dtype, activation_checkpointing=ac_mode))
        return build_parallel_vlm(job, device, device_mesh, transport=transport)
    builder = registry.get("model", model_config.model_type)
    with torch.device(device):  # parameters are drawn on the target device (fp32), then cast
        model = builder(model_config, **({"vlm_config": vlm_config} if vlm_config is not None else {}), **model_kwargs)
    model = model.to(device=device, dtype=param_dtype)
    if hasattr(model, "rope_tables"):
        model.rope_tables(device, 0, 1)

    model._kf_mesh = device_mesh  # checkpoints describe TP / EP shards as sharded tensors over this mesh
    _, tp_size, _ = mesh_dim(device_mesh, "tp")
    if tp_size > 1:
        from kempnerforge_b200.parallel.tensor_parallel import apply_tensor_parallel

        apply_tensor_parallel(model, device_mesh)
    if model_config.is_moe and device_mesh is not None:
        from kempnerforge_b200.parallel.expert_parallel import apply_expert_parallel, ep_group_for

        ep_pg, ep_size = ep_group_for(device_mesh, ep_in_dp)
        if ep_size > 1:
            apply_expert_parallel(model, ep_pg, ep_in_dp)
    if fp8:
        apply_float8(model)
    if ac_mode and str(ac_mode) != "none":
        apply_ac(model, str(ac_mode))
    apply_fsdp2(model, device_mesh, transport=transport, param_sharding=param_sharding)
    if compile_model:
        log.info("compile_model is accepted for preset compatibility; this build has no tracing compiler")
    return model


def build_parallel_vlm(job_config, device: torch.device, device_mesh=None, *, step: int = 0,
                       transport: str | None = None) -> nn.Module:
    """Vision encoder + adapter + transformer as one data-parallel model.

    Order: build -> cast (the transformer and adapter to the training dtype; a frozen encoder keeps its own
    dtype and stays in eval mode) -> freeze according to the schedule at ``step`` -> AC -> sharded DP over
    the trainable parameters only (frozen ones are replicated and never enter a flat group).
    Parity: kempnerforge/distributed/parallel.py:305-496 (VLM variants of the FSDP wrapping).
    """
    from kempnerforge_b200.models.vlm import build_vlm_wrapper, is_encoder_frozen
    from kempnerforge_b200.training.freeze import apply_freeze_specs, effective_freeze

    cfg = job_config
    tc = cfg.train
    frames = cfg.video.max_frames if cfg.video is not None else 1
    with torch.device(device):
        model = build_vlm_wrapper(cfg.model, cfg.vision_encoder, cfg.adapter, cfg.vlm, frames_per_clip=frames)
    model.transformer.to(device=device, dtype=tc.param_dtype)
    model.adapter.to(device=device, dtype=tc.param_dtype)
    specs = effective_freeze(cfg.vlm, step)
    apply_freeze_specs(model, specs, cfg.vlm.module_patterns)
    if is_encoder_frozen(specs):
        model.vision_encoder.to(device=device).eval()
    else:
        model.vision_encoder.to(device=device, dtype=tc.param_dtype)
    model.transformer.rope_tables(device, 0, 1)
    ac = str(tc.activation_checkpointing)
    if ac != "none":
        apply_ac(model, ac)
    apply_fsdp2(model, device_mesh, transport=transport)
    n_train = sum(p.numel() for p in model.parameters() if p.requires_grad)
    n_all = sum(p.numel() for p in model.parameters())
    log.info("VLM (%s): %s trainable of %s parameters", cfg.vlm.arch, f"{n_train:,}", f"{n_all:,}")
    return model
