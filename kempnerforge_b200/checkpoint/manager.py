"""Checkpoint manager: DCP tensor state + ``train_state.pt`` + ``metadata.json`` + a ``latest`` link.

Directory layout (interchangeable with the reference):

    {dir}/step_{N}/.metadata, __{rank}_{k}.distcp     tensors, keys "model.<fqn>" / "optimizer.state.<fqn>.*"
    {dir}/step_{N}/train_state.pt                     counters, RNG, scheduler, data loader (rank 0)
    {dir}/step_{N}/metadata.json                      {"step", "tokens_seen"[, "vlm_freeze"]}
    {dir}/latest -> step_{N}                          committed atomically (symlink + rename)
    {dir}/step_{N}/pp{r}/...                          one sub-directory per pipeline stage

Tensors are written as whole (replicated) tensors, so a checkpoint does not depend on the number
of GPUs that wrote it; sharded optimizer moments are gathered for the save and re-cut on load.

Asynchronous saves commit ``latest`` late: a new save first waits for the previous flush, commits
*that* checkpoint's link, then starts its own flush; ``wait()`` / ``flush_pending_save()`` commit
the last one.  A crash in the middle therefore never leaves ``latest`` pointing at a partial
directory.  Retention (``keep_last_n``) never removes ``latest``'s target, an in-flight directory
or a dynamic-window milestone.  ``train_state.pt`` is a pickle: it is only loaded when the file
belongs to the current user (or root) and is not writable by others.

Parity: kempnerforge/checkpoint/manager.py:44-671.
"""

from __future__ import annotations

import json
import logging
import os
import shutil
import stat
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from kempnerforge_b200.checkpoint.async_save import AsyncCheckpointer
from kempnerforge_b200.checkpoint.state import build_train_state, restore_train_state
from kempnerforge_b200.resilience.elastic import list_step_dirs

log = logging.getLogger(__name__)


class UntrustedCheckpointError(PermissionError, RuntimeError):
    """``train_state.pt`` is a pickle: a file that another user owns is not loaded."""


def check_trusted_file(path: Path) -> None:
    """The trust boundary of ``train_state.pt`` (a full pickle: loading it runs whatever it contains).  A file owned by
    another uid is refused (``PermissionError``); a file that group or others may write is loaded with a warning that
    names the mode, like the reference does (kempnerforge/checkpoint/manager.py:75-110)."""
    st = path.stat()
    uid = os.getuid()
    if st.st_uid != uid:
        raise UntrustedCheckpointError(
            f"Refusing to load {path}: owned by uid={st.st_uid}, current uid={uid}.  The file is a pickle and loading it "
            f"executes arbitrary Python; chown it to the current user after inspection if you trust it.")
    if st.st_mode & (stat.S_IWGRP | stat.S_IWOTH):
        log.warning("%s is group/world-writable (mode=%s): it is a pickle and any writer can inject code that runs at load "
                    "time; consider chmod g-w,o-w on the checkpoint directory", path, oct(st.st_mode & 0o777))


def _intersect_freeze_meta_by_module(saved: list[dict], expected: list[dict]) -> tuple[list[dict], list[dict]]:
    """Both freeze records restricted to the modules that appear in each of them, input order kept.  A checkpoint of
    one vision-language architecture can be resumed into another: modules only one side knows are not compared."""
    shared = {e["module"] for e in saved} & {e["module"] for e in expected}
    return [e for e in saved if e["module"] in shared], [e for e in expected if e["module"] in shared]


def _load_train_state(path: Path) -> dict:
    """Trust check, then the unpickling load of one ``train_state.pt``."""
    check_trusted_file(path)
    return torch.load(path, map_location="cpu", weights_only=False)


# --------------------------------------------------------------------------- state dict assembly
def _unwrap(model):
    return getattr(model, "module", model)


def _shard_meshes(model) -> dict[str, Any]:
    """{"tp": 1-D DeviceMesh, "ep": 1-D DeviceMesh} for the mesh dimensions this model's parameters are sharded over."""
    m = _unwrap(model)
    mesh = getattr(m, "_kf_mesh", None)
    out: dict[str, Any] = {}
    if mesh is None:
        return out
    names = mesh.mesh_dim_names or ()
    if "tp" in names:
        out["tp"] = mesh["tp"]
    if "ep" in names:
        out["ep"] = mesh["ep"]
    elif getattr(m, "ep_in_dp", False) and "dp_shard" in names:
        out["ep"] = mesh["dp_shard"]  # experts sharded over the data-parallel ranks
    return out


def as_sharded(t: torch.Tensor, spec, meshes: dict[str, Any]):
    """Describe a rank-local shard to the checkpoint layer: a DTensor over the 1-D mesh of its parallel dimension,
    so that every rank's piece is written (not just rank 0's) and a different world size can re-shard on load."""
    if spec is None or spec[0] not in meshes:
        return t
    from torch.distributed.tensor import DTensor, Shard

    return DTensor.from_local(t, meshes[spec[0]], [Shard(spec[1])], run_check=False)


def to_local(t):
    return t.to_local() if hasattr(t, "to_local") else t


def _shard_specs(model) -> dict[str, tuple[str, int]]:
    return {n: p._kf_shard for n, p in _unwrap(model).named_parameters(remove_duplicate=False)
            if getattr(p, "_kf_shard", None) is not None}


def model_state_dict(model) -> dict[str, torch.Tensor]:
    engine = getattr(_unwrap(model), "_kf_engine", None)
    if engine is not None and hasattr(engine, "wait_all"):
        engine.wait_all()  # parameters being published asynchronously must have landed
    sd = dict(_unwrap(model).state_dict())
    if engine is not None and getattr(engine, "sharded_groups", None):
        # ZeRO-3 units: ``state_dict`` sees staging memory; the truth is in the shards
        row_mesh = _dp_row_mesh(model, engine)
        names = {id(p): n for n, p in _unwrap(model).named_parameters(remove_duplicate=False)}
        for g in engine.sharded_groups:
            for i, p in enumerate(g.params):
                name = names[id(p)]
                if name not in sd:
                    continue
                if row_mesh is not None and _row_shardable(g, i, p):
                    from torch.distributed.tensor import DTensor, Shard

                    local = g.piece_of(p).view(p.shape[0] // g.world, *p.shape[1:])
                    sd[name] = DTensor.from_local(local, row_mesh, [Shard(0)], run_check=False)
                else:
                    sd[name] = engine.full_parameter(p)
    meshes = _shard_meshes(model)
    if meshes:
        for name, spec in _shard_specs(model).items():
            if name in sd:
                sd[name] = as_sharded(sd[name], spec, meshes)
    return sd


def _row_shardable(g, i: int, p) -> bool:
    """The piece of parameter i of a sharded unit is exactly rows [r * R / N, (r + 1) * R / N) of the parameter."""
    return p.dim() >= 1 and g.padded[i] == p.numel() and p.shape[0] % g.world == 0


def load_model_state_dict(model, loaded: dict[str, Any]) -> None:
    engine = getattr(_unwrap(model), "_kf_engine", None)
    if engine is not None and getattr(engine, "sharded_groups", None):
        loaded = dict(loaded)
        names = {id(p): n for n, p in _unwrap(model).named_parameters(remove_duplicate=False)}
        for g in engine.sharded_groups:
            for i, p in enumerate(g.params):
                v = loaded.pop(names[id(p)], None)
                if v is None:
                    continue
                if hasattr(v, "to_local") and _row_shardable(g, i, p):
                    g.piece_of(p).copy_(v.to_local().reshape(-1))
                else:
                    engine.load_full_parameter(p, v.full_tensor() if hasattr(v, "full_tensor") else v)
            g.valid = set()
        engine._stage_owner = None
        if not engine.shared_staging:
            for g in engine.sharded_groups:
                engine.acquire(g, everything=True)
    _unwrap(model).load_state_dict({k: to_local(v) for k, v in loaded.items()}, strict=False)


def _param_fqns(model) -> dict[int, str]:
    return {id(p): n for n, p in _unwrap(model).named_parameters(remove_duplicate=False)}


def _dp_row_mesh(model, engine):
    """The 1-D data-parallel mesh over which flat moment shards can be described as row shards, or None.

    Flat shards cut parameters at arbitrary elements, which no sharded-tensor placement can express.  When the
    engine's group is exactly the ``dp_shard`` mesh dimension, every rank instead keeps rows [r*R/N, (r+1)*R/N) of
    each parameter's moments and hands them to the checkpoint layer as ``Shard(0)`` over that mesh: the layout the
    reference's FSDP2 optimizer state has (kempnerforge/checkpoint/state.py, DTensor shards over ``dp_shard``), with
    1/N of the moments per rank instead of a full copy on every rank."""
    if engine is None or engine.world <= 1:
        return None
    mesh = getattr(_unwrap(model), "_kf_mesh", None)
    names = (mesh.mesh_dim_names or ()) if mesh is not None else ()
    if "dp_shard" not in names or mesh["dp_shard"].size() != engine.world:
        return None
    return mesh["dp_shard"]


def _rows_of(full: torch.Tensor, shape, rank: int, world: int) -> torch.Tensor:
    rows = shape[0] // world
    return full.view(shape)[rank * rows : (rank + 1) * rows].clone()


def optimizer_state_dict(model, optimizer) -> dict[str, Any]:
    """{"state": {fqn: {...}}, "param_groups": [{"params": [fqn...], ...}]}; flat moments of a data-parallel run
    appear as row shards over the ``dp_shard`` mesh (one unit is assembled at a time, then cut and released)."""
    fqn_of = _param_fqns(model)
    engine = getattr(_unwrap(model), "_kf_engine", None)
    opts = [optimizer] + ([optimizer.inner_adam] if getattr(optimizer, "inner_adam", None) is not None else [])
    state: dict[str, dict] = {}
    groups = []
    row_mesh = _dp_row_mesh(model, engine)
    specs = _shard_specs(model) if row_mesh is not None else {}
    for opt in opts:
        flat_groups = getattr(opt, "_flat_groups", None) or []
        flat_param_ids = set()
        for fg in flat_groups:
            if getattr(fg, "sharded", False):
                for i, p in enumerate(fg.params):
                    flat_param_ids.add(id(p))
                    lo, hi = fg.offsets[i] // fg.world, (fg.offsets[i] + fg.padded[i]) // fg.world
                    entry = {"step": fg.step_tensor.detach().clone().cpu()}
                    for key, buf in (("exp_avg", fg.exp_avg), ("exp_avg_sq", fg.exp_avg_sq)):
                        piece = buf[lo:hi]
                        if row_mesh is not None and _row_shardable(fg, i, p):
                            from torch.distributed.tensor import DTensor, Shard

                            entry[key] = DTensor.from_local(piece.view(p.shape[0] // fg.world, *p.shape[1:]), row_mesh,
                                                            [Shard(0)], run_check=False)
                        else:
                            full = torch.empty(fg.padded[i], dtype=buf.dtype, device=buf.device)
                            dist.all_gather_into_tensor(full, piece.contiguous(), group=engine.pg)
                            entry[key] = full[: p.numel()].view(p.shape).clone()
                    state[fqn_of[id(p)]] = entry
                continue
            if engine is not None and engine.world > 1:
                m_full, v_full = engine.full_optimizer_state(fg)
            else:
                m_full, v_full = fg.exp_avg, fg.exp_avg_sq
            for p, off in zip(fg.params, fg.offsets):
                flat_param_ids.add(id(p))
                fqn = fqn_of[id(p)]
                m_p, v_p = m_full[off : off + p.numel()], v_full[off : off + p.numel()]
                if (row_mesh is not None and not fg.local and fqn not in specs and p.dim() >= 1
                        and p.shape[0] % engine.world == 0 and p.shape[0] >= engine.world):
                    from torch.distributed.tensor import DTensor, Shard

                    m_p = DTensor.from_local(_rows_of(m_p, p.shape, engine.rank, engine.world), row_mesh, [Shard(0)], run_check=False)
                    v_p = DTensor.from_local(_rows_of(v_p, p.shape, engine.rank, engine.world), row_mesh, [Shard(0)], run_check=False)
                else:
                    m_p, v_p = m_p.view(p.shape), v_p.view(p.shape)
                    if m_full is not fg.exp_avg:  # do not keep the whole gathered unit alive through a view
                        m_p, v_p = m_p.clone(), v_p.clone()
                state[fqn] = {"step": fg.step_tensor.detach().clone().cpu(), "exp_avg": m_p, "exp_avg_sq": v_p}
            del m_full, v_full
        for p, st in opt.state.items():
            if id(p) in flat_param_ids or id(p) not in fqn_of:
                continue
            state[fqn_of[id(p)]] = {
                k: (v.to_local() if hasattr(v, "to_local") else v) if torch.is_tensor(v) else torch.tensor(float(v))
                for k, v in st.items()
            }
        for g in opt.param_groups:
            groups.append({**{k: v for k, v in g.items() if k != "params"},
                           "params": [fqn_of[id(p)] for p in g["params"] if id(p) in fqn_of]})
    meshes = _shard_meshes(model)
    if meshes:
        specs = _shard_specs(model)
        params = dict(_unwrap(model).named_parameters(remove_duplicate=False))
        for fqn, entry in state.items():
            spec = specs.get(fqn)
            if spec is None:
                continue
            for k, v in entry.items():
                if torch.is_tensor(v) and v.dim() > 0 and v.shape == params[fqn].shape:
                    entry[k] = as_sharded(v.contiguous(), spec, meshes)
    return {"state": state, "param_groups": groups}


def _whole(v, model_sharded: bool):
    """A loaded state tensor as this rank needs it: the local part of a tensor- / expert-parallel shard (the
    parameter itself is sharded that way), the whole tensor for row shards of a data-parallel moment, else itself."""
    if not hasattr(v, "to_local"):
        return v
    return v.to_local() if model_sharded else v.full_tensor()


def load_optimizer_state_dict(model, optimizer, loaded: dict[str, Any]) -> None:
    """Inverse of ``optimizer_state_dict`` for tensors that were loaded in place (flat views) or into copies."""
    specs = _shard_specs(model)
    # moments of ZeRO-3 units stay row shards (the local rows go straight into the shard-layout buffers)
    keep_rows = set()
    eng0 = getattr(_unwrap(model), "_kf_engine", None)
    if eng0 is not None and getattr(eng0, "sharded_groups", None):
        fq = _param_fqns(model)
        keep_rows = {fq[id(p)] for g in eng0.sharded_groups for i, p in enumerate(g.params) if _row_shardable(g, i, p)}
    loaded = {**loaded, "state": {fqn: {k: (to_local(v) if fqn in keep_rows and k in ("exp_avg", "exp_avg_sq") and
                                            hasattr(v, "to_local") else _whole(v, fqn in specs))
                                        for k, v in entry.items()}
                                  for fqn, entry in loaded["state"].items()}}
    name_to_param = dict(_unwrap(model).named_parameters(remove_duplicate=False))
    engine = getattr(_unwrap(model), "_kf_engine", None)
    opts = [optimizer] + ([optimizer.inner_adam] if getattr(optimizer, "inner_adam", None) is not None else [])
    handled = set()
    for opt in opts:
        for fg in getattr(opt, "_flat_groups", None) or []:
            if getattr(fg, "sharded", False):
                fqn_of = _param_fqns(model)
                step = None
                for i, p in enumerate(fg.params):
                    entry = loaded["state"].get(fqn_of[id(p)])
                    handled.add(fqn_of[id(p)])
                    if entry is None:
                        continue
                    piece = fg.padded[i] // fg.world
                    lo = fg.offsets[i] // fg.world
                    for key, buf in (("exp_avg", fg.exp_avg), ("exp_avg_sq", fg.exp_avg_sq)):
                        flat = entry[key].reshape(-1)
                        if flat.numel() == piece and piece != p.numel():   # this rank's rows of a row-sharded moment
                            buf[lo : lo + piece].copy_(flat)
                            continue
                        a, b = fg.rank * piece, min((fg.rank + 1) * piece, flat.numel())   # a whole tensor
                        buf[lo : lo + piece].zero_()
                        if b > a:
                            buf[lo : lo + b - a].copy_(flat[a:b])
                    step = entry.get("step", step)
                if step is not None:
                    fg.load_step(int(float(step)))
                continue
            full_m = torch.zeros(fg.numel, dtype=fg.exp_avg.dtype, device=fg.exp_avg.device)
            full_v = torch.zeros_like(full_m)
            step = None
            fqn_of = _param_fqns(model)
            for p, off in zip(fg.params, fg.offsets):
                entry = loaded["state"].get(fqn_of[id(p)])
                handled.add(fqn_of[id(p)])
                if entry is None:
                    continue
                full_m[off : off + p.numel()].copy_(entry["exp_avg"].reshape(-1))
                full_v[off : off + p.numel()].copy_(entry["exp_avg_sq"].reshape(-1))
                step = entry.get("step", step)
            lo, hi = fg.shard_range
            fg.exp_avg.copy_(full_m[lo:hi])
            fg.exp_avg_sq.copy_(full_v[lo:hi])
            if step is not None:
                fg.load_step(int(float(step)))
        owned = {id(p) for g in opt.param_groups for p in g["params"]}
        for fqn, entry in loaded["state"].items():
            p = name_to_param.get(fqn)
            if fqn in handled or p is None or id(p) not in owned:
                continue
            dst = opt.state[p]
            for k, v in entry.items():
                if torch.is_tensor(v) and v.dim() > 0:
                    cur = dst.get(k)
                    if torch.is_tensor(cur) and cur.shape == v.shape:
                        (cur.to_local() if hasattr(cur, "to_local") else cur).copy_(v)
                    else:
                        dst[k] = v.to(p.device)
                elif k in ("weight_sum",):
                    dst[k] = float(v)
                elif k == "k":
                    dst[k] = int(float(v))
                else:
                    dst[k] = v if torch.is_tensor(v) else torch.tensor(float(v))
            handled.add(fqn)
    # hyper-parameters travel with the groups (the scheduled lr above all): groups are matched by position
    saved_groups = list(loaded.get("param_groups", []))
    live_groups = [g for opt in opts for g in opt.param_groups]
    if len(saved_groups) == len(live_groups):
        for live, saved in zip(live_groups, saved_groups):
            for k, v in saved.items():
                if k != "params" and k in live:
                    live[k] = tuple(v) if isinstance(live[k], tuple) and isinstance(v, list) else v
    if hasattr(optimizer, "_k"):
        ks = [int(st["k"]) for st in optimizer.state.values() if "k" in st]
        if ks:
            optimizer._k = max(ks)


def _optimizer_template(model, optimizer) -> dict[str, Any]:
    """Freshly allocated tensors of the right shapes for ``dcp.load`` to fill."""
    tmpl = optimizer_state_dict(model, optimizer)
    for fqn, entry in tmpl["state"].items():
        tmpl["state"][fqn] = {k: (_clone_like(v) if torch.is_tensor(v) else v) for k, v in entry.items()}
    return tmpl


def _clone_like(v: torch.Tensor) -> torch.Tensor:
    if hasattr(v, "to_local"):
        from torch.distributed.tensor import DTensor

        return DTensor.from_local(v.to_local().detach().clone(), v.device_mesh, v.placements, run_check=False)
    return v.detach().clone()


def materialize_optimizer_state(model, optimizer) -> None:
    """Create empty per-parameter state (as a first ``step`` would) so a template exists before loading."""
    for opt in [optimizer] + ([optimizer.inner_adam] if getattr(optimizer, "inner_adam", None) is not None else []):
        flat_ids = {id(p) for fg in (getattr(opt, "_flat_groups", None) or []) for p in fg.params}
        name = type(opt).__name__
        for g in opt.param_groups:
            for p in g["params"]:
                if not p.requires_grad or id(p) in flat_ids or len(opt.state[p]) > 0:
                    continue
                if name in ("FusedAdamW", "AdamW"):
                    opt.state[p] = {"step": torch.zeros((), dtype=torch.float32, device=p.device),
                                    "exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)}
                elif name == "Lion":
                    opt.state[p] = {"exp_avg": torch.zeros_like(p)}
                elif name == "Muon":
                    opt.state[p] = {"momentum_buffer": torch.zeros_like(p)}
                elif name == "ScheduleFreeAdamW":
                    opt.state[p] = {"z": p.detach().clone(), "v": torch.zeros_like(p), "x": p.detach().clone(),
                                    "weight_sum": 0.0, "k": 0}


# --------------------------------------------------------------------------- manager
class CheckpointManager:
    def __init__(self, config, model, optimizer, process_group=None, pp_rank: int | None = None) -> None:
        self.config = config
        self.model = model
        self.optimizer = optimizer
        self.pp_rank = pp_rank
        self.dir = Path(config.dir)
        self.process_group = process_group
        self._dist = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank() if self._dist else 0
        self.group_rank = dist.get_rank(process_group) if (self._dist and process_group is not None) else self.rank
        self._sync_group = None
        if self._dist and dist.get_world_size() > 1:
            # a dedicated gloo group: barriers issued from the main thread must not interleave with the
            # collectives DCP issues from its background thread on the default group
            self._sync_group = dist.new_group(backend="gloo")
        self._saver = AsyncCheckpointer(str(config.async_mode), process_group)
        if self._saver.is_async and self._dist and dist.get_world_size() > 1 and process_group is None:
            # the background flush exchanges its plans through collectives of its own: on the default group they would
            # run concurrently with the training step's (and this manager's) collectives issued by the main thread
            self._saver.process_group = dist.new_group(backend="gloo")
        self._pending_finalize: tuple[Path, int] | None = None
        self._stashed_dataloader_state: dict | None = None

    # ------------------------------------------------------------------ paths
    def step_dir(self, step: int) -> Path:
        return self.dir / f"step_{step}"

    def _dcp_dir(self, step_dir: Path) -> Path:
        return step_dir / f"pp{self.pp_rank}" if self.pp_rank is not None else step_dir

    def _is_writer(self) -> bool:
        return self.rank == 0

    def _barrier(self) -> None:
        if self._sync_group is not None:
            dist.barrier(group=self._sync_group)

    def _commit_latest(self, step_dir: Path, step: int) -> None:
        if self._is_writer():
            tmp = self.dir / "latest.tmp"
            if tmp.is_symlink() or tmp.exists():
                tmp.unlink()
            tmp.symlink_to(step_dir.name)
            os.replace(tmp, self.dir / "latest")
            log.info("Checkpoint committed: %s (step=%d)", step_dir, step)
            log.info("Checkpoint saved: %s (step=%d)", step_dir, step)

    def _drain_pending_finalize(self) -> None:
        if self._pending_finalize is not None:
            step_dir, step = self._pending_finalize
            self._pending_finalize = None
            self._commit_latest(step_dir, step)
            self._cleanup()

    # ------------------------------------------------------------------ save
    def save(self, step: int, tokens_seen: int = 0, scheduler=None, dataloader=None, extra: dict | None = None) -> Path:
        step_dir = self.step_dir(step)
        dcp_dir = self._dcp_dir(step_dir)
        dcp_dir.mkdir(parents=True, exist_ok=True)
        # the previous flush must be over before this save issues collectives of its own (gathering sharded moments)
        self._saver.wait()
        # an optimizer that has not stepped yet (a save at step 0) gets its zero state first, so that every checkpoint
        # carries the full set of keys a later load asks for
        materialize_optimizer_state(self.model, self.optimizer)
        state = {"model": model_state_dict(self.model), "optimizer": optimizer_state_dict(self.model, self.optimizer)}
        self._saver.save(state, str(dcp_dir), self.process_group)  # waits for the previous flush first
        self._drain_pending_finalize()
        if self._is_writer() or (self.pp_rank is not None and self.group_rank == 0):
            train_state = build_train_state(step, tokens_seen, scheduler, dataloader, extra)
            if self._is_writer():  # the reference's layout: one train state per step, written by rank 0
                torch.save(train_state, step_dir / "train_state.pt")
            if self.pp_rank is not None and self.group_rank == 0:  # plus one per stage (its own RNG / loader state)
                torch.save(train_state, dcp_dir / "train_state.pt")
        if self._is_writer():
            meta = {"step": step, "tokens_seen": tokens_seen}
            if extra and "vlm_freeze" in extra:
                meta["vlm_freeze"] = extra["vlm_freeze"]
            (step_dir / "metadata.json").write_text(json.dumps(meta))
        if self._saver.is_async:
            self._pending_finalize = (step_dir, step)
        else:
            self._barrier()
            self._commit_latest(step_dir, step)
            self._cleanup()
        self._barrier()
        return step_dir

    def wait(self) -> None:
        """Block until the in-flight save (if any) is on disk and committed."""
        self._saver.wait()
        self._barrier()
        self._drain_pending_finalize()
        self._barrier()

    flush_pending_save = wait

    def peek_saved_step(self, path: str | Path | None = None) -> int | None:
        """Step number recorded in a checkpoint's metadata without loading tensors."""
        target = self._resolve_load_path(path)
        if target is None:
            return None
        meta = target / "metadata.json"
        if meta.exists():
            try:
                return int(json.loads(meta.read_text())["step"])
            except (ValueError, KeyError):
                return None
        return None

    # ------------------------------------------------------------------ load
    def _resolve_load_path(self, path) -> Path | None:
        for cand in (path, self.config.load_path):
            if cand:
                p = Path(cand)
                if p.name == "latest" or p.is_symlink():
                    p = p.resolve()
                return p if p.exists() else None
        latest = self.dir / "latest"
        if latest.exists():
            return latest.resolve()
        steps = list_step_dirs(self.dir)
        return steps[-1][1] if steps else None

    def _resolve_dcp_load_dir(self, step_dir: Path) -> Path | None:
        """``step_dir`` if its tensor data is complete, else the newest earlier checkpoint that is."""
        def complete(d: Path) -> bool:
            return (self._dcp_dir(d) / ".metadata").exists()

        if complete(step_dir):
            return step_dir
        log.warning("checkpoint %s is incomplete (no .metadata); looking for an older complete one", step_dir)
        for _, cand in reversed(list_step_dirs(step_dir.parent)):
            if cand != step_dir and complete(cand):
                return cand
        return None

    def load(self, path=None, scheduler=None, dataloader=None, exclude_keys: list[str] | None = None,
             vlm_freeze_expected: list[dict] | None = None, allow_fallback: bool | None = None) -> tuple[int, int, dict]:
        """Restore model / optimizer / train state; returns (step, tokens_seen, extras) — (0, 0, {}) if nothing found.

        An incomplete checkpoint (tensor data without ``.metadata``) is replaced by the newest complete one only on
        auto-resume (``allow_fallback``; default: no explicit ``path`` and no ``checkpoint.load_path``).  An explicit
        path is honoured as given and fails loudly, like the reference; rank 0 decides and the others follow."""
        if allow_fallback is None:
            allow_fallback = not path and not self.config.load_path
        step_dir = self._resolve_load_path(path)
        exists = step_dir is not None
        if self._dist and dist.get_world_size() > 1:  # rank 0's view of the filesystem is authoritative
            box = [str(step_dir) if exists else ""]
            dist.broadcast_object_list(box, src=0, group=self._sync_group)
            step_dir, exists = (Path(box[0]), True) if box[0] else (None, False)
        if not exists:
            asked = path or self.config.load_path
            if asked:
                log.warning("checkpoint path %s does not exist; starting from scratch", asked)
            else:
                log.info("no checkpoint found under %s; starting from scratch", self.dir)
            return 0, 0, {}
        exclude = set(exclude_keys or [])
        wants_tensors = not {"model", "optimizer"} <= exclude
        if wants_tensors and allow_fallback:
            chosen = self._resolve_dcp_load_dir(step_dir)
            if self._dist and dist.get_world_size() > 1:
                box = [str(chosen) if chosen is not None else ""]
                dist.broadcast_object_list(box, src=0, group=self._sync_group)
                chosen = Path(box[0]) if box[0] else None
            if chosen is None:
                log.warning("no complete checkpoint available; starting from scratch")
                return 0, 0, {}
            step_dir = chosen
        self._check_freeze_metadata(step_dir, vlm_freeze_expected)
        state: dict[str, Any] = {}
        if "model" not in exclude:
            state["model"] = model_state_dict(self.model)
        if "optimizer" not in exclude:
            materialize_optimizer_state(self.model, self.optimizer)
            state["optimizer"] = _optimizer_template(self.model, self.optimizer)
        if state:
            if "optimizer" in state:
                self._drop_unsaved_group_fields(state["optimizer"], self._dcp_dir(step_dir))
            dcp.load(state, checkpoint_id=str(self._dcp_dir(step_dir)), process_group=self.process_group)
            if "model" in state:
                load_model_state_dict(self.model, state["model"])
            if "optimizer" in state:
                load_optimizer_state_dict(self.model, self.optimizer, state["optimizer"])
        train_state = self._load_train_state(step_dir)
        if train_state is None:
            return self._step_from_name(step_dir), 0, {}
        if dataloader is None and "dataloader" in train_state:
            self._stashed_dataloader_state = train_state["dataloader"]
        step, tokens, extra = restore_train_state(train_state, scheduler, dataloader)
        log.info("Checkpoint loaded: %s (step=%d)", step_dir, step)
        return step, tokens, extra

    @staticmethod
    def _drop_unsaved_group_fields(opt_state: dict, dcp_dir: Path) -> None:
        """Hyper-parameter fields of the live param groups that the checkpoint does not contain (for instance
        ``initial_lr``, which only exists once a scheduler has been attached) keep their current values instead of
        failing the load.  The same goes for per-parameter state of a checkpoint written before the optimizer's first
        step: the freshly created zero state stays."""
        try:
            saved = set(dcp.FileSystemReader(str(dcp_dir)).read_metadata().state_dict_metadata)
        except Exception:  # unreadable metadata is reported by dcp.load itself
            return
        if not any(k.startswith("optimizer.state.") for k in saved):
            if opt_state.get("state"):
                log.warning("checkpoint %s has no optimizer state (saved before the first step): moments start at zero",
                            dcp_dir)
            opt_state["state"] = {}
        for i, group in enumerate(opt_state.get("param_groups", [])):
            for key in [k for k in group if k != "params"]:
                if f"optimizer.param_groups.{i}.{key}" not in saved:
                    log.info("checkpoint has no optimizer.param_groups.%d.%s; keeping the current value", i, key)
                    del group[key]

    @staticmethod
    def _step_from_name(step_dir: Path) -> int:
        try:
            return int(step_dir.name.split("_")[1])
        except (IndexError, ValueError):
            return 0

    def _load_train_state(self, step_dir: Path) -> dict | None:
        target = (self._dcp_dir(step_dir) if self.pp_rank is not None else step_dir) / "train_state.pt"
        if self.pp_rank is not None and not target.exists() and (step_dir / "train_state.pt").exists():
            # a checkpoint in the reference's layout: one train state for all stages
            log.info("no per-stage train state in %s; reading %s", target.parent, step_dir / "train_state.pt")
            target = step_dir / "train_state.pt"
        multi = self._dist and dist.get_world_size() > 1 and self.pp_rank is None
        state = None
        if not multi or self.rank == 0:
            if target.exists():
                state = _load_train_state(target)
        if multi:
            box = [state]
            dist.broadcast_object_list(box, src=0, group=self._sync_group)
            state = box[0]
        return state

    def _check_freeze_metadata(self, step_dir: Path, expected: list[dict] | None) -> None:
        if expected is None:
            return
        meta_path = step_dir / "metadata.json"
        if not meta_path.exists():
            return
        try:
            saved = json.loads(meta_path.read_text()).get("vlm_freeze")
        except (OSError, ValueError, AttributeError) as e:
            log.warning("could not read %s (%s): freeze configuration not compared", meta_path, e)
            return
        if saved is None:
            return
        saved_shared, want_shared = _intersect_freeze_meta_by_module(saved, expected)
        pairs = lambda meta: {(e["module"], bool(e["frozen"])) for e in meta}  # noqa: E731  order carries no meaning
        if pairs(saved_shared) != pairs(want_shared):
            only_saved = sorted({e["module"] for e in saved} - {e["module"] for e in expected})
            only_now = sorted({e["module"] for e in expected} - {e["module"] for e in saved})
            note = f" (cross-arch keys ignored, known to one side only: saved-only={only_saved}, current-only={only_now})" \
                if only_saved or only_now else ""
            msg = f"VLM freeze mismatch at {step_dir}: saved={saved_shared}, current={want_shared}{note}"
            if self.config.ignore_freeze_mismatch:
                log.warning(msg)
            else:
                raise ValueError(msg + " (set checkpoint.ignore_freeze_mismatch=true to continue)")

    def apply_dataloader_state(self, dataloader) -> None:
        """Hand a data-loader state that was loaded before the loader existed over to the loader.  The state is dropped
        afterwards in every case (a loader without ``load_state_dict``, or none, cannot take it later either)."""
        state, self._stashed_dataloader_state = self._stashed_dataloader_state, None
        if state is not None and dataloader is not None and hasattr(dataloader, "load_state_dict"):
            dataloader.load_state_dict(state)

    # ------------------------------------------------------------------ retention
    def _cleanup(self) -> None:
        keep = self.config.keep_last_n
        if keep is None or keep <= 0 or not self._is_writer():
            return
        steps = list_step_dirs(self.dir)
        protected = set()
        latest = self.dir / "latest"
        if latest.exists():
            protected.add(latest.resolve())
        if self._pending_finalize is not None:
            protected.add(self._pending_finalize[0].resolve())
        regular = [(s, d) for s, d in steps if not self.config.is_dynamic_milestone(s)]
        for s, d in regular[:-keep] if len(regular) > keep else []:
            if d.resolve() in protected:
                continue
            shutil.rmtree(d, ignore_errors=True)
            log.info("removed old checkpoint %s", d)
