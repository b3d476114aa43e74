"""Process-group bootstrap and the device mesh.

One process per GPU.  Rank information comes from the torchrun variables with a SLURM
fallback; the mesh lists only dimensions larger than one, in the fixed order
(pp, dp_replicate, dp_shard, ep, tp) so tensor-parallel peers are NVLink neighbours and
pipeline stages are outermost; a size-1 ``dp_shard`` dimension is kept whenever TP or EP is
active so the sharding code always finds a data-parallel mesh.  On CPU-only hosts the same
code runs with the gloo backend and a "cpu" mesh.

Parity: kempnerforge/distributed/setup.py:24-273 (world info, NCCL environment policy,
timed barrier, seed + pp_rank, mesh dimension order and names, single-process shortcut).
"""

from __future__ import annotations

import logging
import os
import random
import socket
import subprocess
from datetime import timedelta

import numpy as np
import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

from kempnerforge_b200.config.sections import DistributedConfig

log = logging.getLogger(__name__)
MESH_DIM_ORDER = ("pp", "dp_replicate", "dp_shard", "ep", "tp")


def get_world_info() -> tuple[int, int, int]:
    """(rank, local_rank, world_size) from torchrun variables, else SLURM, else a single process.  The three standard
    variables are exported when they were missing, so that an ``env://`` rendezvous started under ``srun`` finds them."""
    env = os.environ
    if "RANK" in env:
        info = int(env["RANK"]), int(env.get("LOCAL_RANK", 0)), int(env.get("WORLD_SIZE", 1))
    elif "SLURM_PROCID" in env:
        info = int(env["SLURM_PROCID"]), int(env.get("SLURM_LOCALID", 0)), int(env.get("SLURM_NTASKS", 1))
    else:
        info = 0, 0, 1
    for key, value in zip(("RANK", "LOCAL_RANK", "WORLD_SIZE"), info):
        env.setdefault(key, str(value))
    return info


def is_rank_zero() -> bool:
    return get_world_info()[0] == 0


def _detect_ib_interface() -> str | None:
    try:
        out = subprocess.run(["ip", "-br", "addr"], capture_output=True, text=True, timeout=5).stdout
    except (OSError, subprocess.SubprocessError):
        return None
    for line in out.splitlines():
        parts = line.split()
        if len(parts) >= 3 and parts[0].startswith("ib") and parts[1] == "UP":
            return parts[0]
    return None


def _set_nccl_env() -> None:
    """Defaults only: anything the user exported wins.  NCCL and Gloo are bound to the same interface (the one the
    user named for NCCL, else the first InfiniBand interface that is up); the InfiniBand / GPUDirect defaults are set
    whether or not such an interface was found; TORCH_NCCL_ASYNC_ERROR_HANDLING defaults to 1 and an explicit 0 is
    kept but warned about (process-group timeouts are then advisory)."""
    env = os.environ
    iface = env.get("NCCL_SOCKET_IFNAME") or _detect_ib_interface()
    if iface:
        env.setdefault("NCCL_SOCKET_IFNAME", iface)
        env.setdefault("GLOO_SOCKET_IFNAME", iface)
    env.setdefault("NCCL_IB_DISABLE", "0")
    env.setdefault("NCCL_NET_GDR_LEVEL", "2")
    if env.get("TORCH_NCCL_ASYNC_ERROR_HANDLING") == "0":
        log.warning("TORCH_NCCL_ASYNC_ERROR_HANDLING=0 detected: NCCL timeouts are advisory, a stuck collective can hang "
                    "for ever")
    else:
        env.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")


def barrier_with_timeout(timeout_sec: float = 60.0, group=None, reason: str = "") -> None:
    """A barrier that raises RuntimeError instead of hanging when a rank never arrives; ``reason`` names the caller
    in the message (a timeout surfaces either as a False return or as an exception from the wait)."""
    what = f"barrier ({reason})" if reason else "barrier"
    work = dist.barrier(async_op=True) if group is None else dist.barrier(group=group, async_op=True)
    if work is None:
        return
    try:
        arrived = work.wait(timeout=timedelta(seconds=timeout_sec))
    except RuntimeError as exc:
        raise RuntimeError(f"{what} failed after at most {timeout_sec}s: {exc}") from exc
    if arrived is False:
        raise RuntimeError(f"{what} timed out after {timeout_sec}s")


_barrier_with_timeout = barrier_with_timeout


def set_seed(seed: int, pp_rank: int = 0) -> None:
    """Same seed on every data/tensor-parallel rank; pipeline stages differ (they hold different layers)."""
    s = seed + pp_rank
    random.seed(s)
    np.random.seed(s % (2**32))
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(s)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("", 0))
        return s.getsockname()[1]


def _resolve_master() -> None:
    env = os.environ
    if "MASTER_ADDR" not in env:
        addr = "127.0.0.1"
        nodelist = env.get("SLURM_JOB_NODELIST")
        if nodelist:
            try:
                out = subprocess.run(["scontrol", "show", "hostnames", nodelist], capture_output=True,
                                     text=True, timeout=10).stdout.split()
                if out:
                    addr = out[0]
            except (OSError, subprocess.SubprocessError):
                pass
        env["MASTER_ADDR"] = addr
    if "MASTER_PORT" not in env:
        job = env.get("SLURM_JOB_ID")
        env["MASTER_PORT"] = str(random.Random(int(job)).randint(20000, 60000) if job else _free_port())


def mesh_shape(config: DistributedConfig, world_size: int) -> tuple[tuple[int, ...], tuple[str, ...]]:
    """Sizes and names of the mesh dimensions for ``world_size`` ranks (pure function)."""
    cfg = config.resolve(world_size)
    sizes = {
        "pp": cfg.pp,
        "dp_replicate": cfg.dp_replicate,
        "dp_shard": cfg.dp_shard,
        "ep": 1 if cfg.ep_in_dp else cfg.ep,
        "tp": cfg.tp,
    }
    names = [n for n in MESH_DIM_ORDER if sizes[n] > 1]
    if (cfg.tp > 1 or sizes["ep"] > 1) and "dp_shard" not in names:
        names = [n for n in MESH_DIM_ORDER if sizes[n] > 1 or n == "dp_shard"]
    if not names:
        names = ["dp_shard"]
    return tuple(sizes[n] for n in names), tuple(names)


def init_distributed(config: DistributedConfig, seed: int = 42) -> DeviceMesh | None:
    """Initialise the process group and return the device mesh (None for a single process)."""
    rank, local_rank, world = get_world_info()
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local_rank % torch.cuda.device_count())
    if world == 1:
        set_seed(seed)
        return None
    _set_nccl_env()
    _resolve_master()
    if not dist.is_initialized():
        backend = config.backend if use_cuda else "gloo"
        kwargs = {}
        if use_cuda:
            kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=timedelta(seconds=config.nccl_timeout_sec), **kwargs)
    sizes, names = mesh_shape(config, world)
    mesh = init_device_mesh("cuda" if use_cuda else "cpu", sizes, mesh_dim_names=names)
    barrier_with_timeout(60.0)
    pp_rank = mesh["pp"].get_local_rank() if "pp" in names else 0
    set_seed(seed, pp_rank)
    log.info("mesh %s %s", names, sizes)
    return mesh


def destroy_distributed() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


def mesh_dim(mesh: DeviceMesh | None, name: str):
    """(process group, size, local rank) of a mesh dimension, or (None, 1, 0) when it is absent."""
    if mesh is None or name not in (mesh.mesh_dim_names or ()):
        return None, 1, 0
    sub = mesh[name]
    return sub.get_group(), sub.size(), sub.get_local_rank()


def has_dp_mesh(device_mesh: DeviceMesh | None) -> bool:
    return device_mesh is not None and any(n in (device_mesh.mesh_dim_names or ()) for n in ("dp_shard", "dp_replicate"))


def get_dp_info(device_mesh: DeviceMesh | None) -> tuple[int, int]:
    """(dp_rank, dp_size) for data loading: only dp_replicate x dp_shard count, never tp / pp / ep."""
    if device_mesh is None:
        return 0, 1
    names = device_mesh.mesh_dim_names or ()
    rank, size = 0, 1
    for n in ("dp_replicate", "dp_shard"):
        if n in names:
            sub = device_mesh[n]
            rank = rank * sub.size() + sub.get_local_rank()
            size *= sub.size()
    return rank, size


def _set_seed(seed: int, rank: int = 0, pp_rank: int = 0) -> None:
    """The reference's spelling: ``rank`` is accepted and ignored (every data / tensor-parallel rank shares the seed)."""
    set_seed(seed, pp_rank)
