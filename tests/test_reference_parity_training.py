"""The CPU plumbing configuration (dim 256, 4 layers, 4 / 2 heads, SwiGLU 688, vocab 1024, batch 4 x 128, AdamW
3e-4 / (0.9, 0.95) / wd 0.1, cosine with 5 warm-up steps, 20 steps) trained here and with the unmodified reference
library from ``baseline/_ref``: same initial weights, same token stream, step-by-step loss and gradient-norm
parity, then identical weights after a checkpoint round trip.  Skipped when the reference is not installed."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REF / "kempnerforge").is_dir(), reason="reference package not installed")

PRESET = str(ROOT / "configs" / "train" / "cpu_plumbing.toml")


def _batches(n, vocab=1024, batch=4, seq=128):
    g = torch.Generator().manual_seed(0)
    out = []
    for _ in range(n):
        tok = torch.randint(0, vocab, (batch, seq + 1), generator=g)
        out.append((tok[:, :-1].contiguous(), tok[:, 1:].contiguous()))     # labels = inputs shifted by one
    return out


def _reference_run(batches, init_out: dict, overrides=()):
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    from kempnerforge.config.loader import load_config
    from kempnerforge.distributed.utils import clip_grad_norm_
    from kempnerforge.model.transformer import Transformer
    from kempnerforge.training.loss import build_loss_fn
    from kempnerforge.training.optimizer import build_optimizer
    from kempnerforge.training.scheduler import build_scheduler

    cfg = load_config(PRESET, list(overrides))
    torch.manual_seed(0)
    model = Transformer(cfg.model)
    mc = cfg.model
    init_out.update({k: v.detach().clone() for k, v in model.state_dict().items()})
    opt = build_optimizer(model, cfg.optimizer)
    sched = build_scheduler(opt, cfg.scheduler, max_steps=cfg.train.max_steps)
    loss_fn = build_loss_fn(cfg.train)
    traj = []
    for ids, labels in batches:          # the reference's text step: forward, loss, backward, clip, step, schedule
        loss = loss_fn(model(ids), labels)
        if mc.num_experts > 0:           # the auxiliary terms the reference's training script adds for MoE models
            loss = loss + mc.moe_aux_loss_weight * model.get_moe_aux_loss()
            if mc.moe_router_z_loss_weight > 0:
                loss = loss + mc.moe_router_z_loss_weight * model.get_moe_router_z_loss()
        loss.backward()
        norm = clip_grad_norm_(model, cfg.train.grad_clip_norm)
        lr = opt.param_groups[0]["lr"]
        opt.step()
        sched.step()
        opt.zero_grad()
        traj.append((float(loss), float(norm), lr))
    return traj, {k: v.detach().clone() for k, v in model.state_dict().items()}


def test_twenty_steps_match_the_reference_and_survive_a_checkpoint_round_trip(tmp_path, monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    from kempnerforge_b200.config import load_config
    from kempnerforge_b200.training.trainer import Trainer

    batches = _batches(20)
    init: dict = {}
    ref_traj, ref_final = _reference_run(batches, init)

    cfg = load_config(PRESET, [f"--checkpoint.dir={tmp_path / 'ck'}", "--metrics.log_interval=1000"])
    t = Trainer(cfg, init_dist=False)
    assert set(t.model.state_dict()) == set(init)
    t.model.load_state_dict(init)                                     # same starting point as the reference
    t.setup_checkpointing()
    ours = []
    for i, (ids, labels) in enumerate(batches):
        if i == 10:                                                   # save, rebuild everything, resume
            t.step = 10
            t.save_checkpoint()
            t.ckpt.wait()
            t = Trainer(cfg, init_dist=False)
            t.setup_checkpointing()
            assert t.step == 10
        out = t.train_step([{"input_ids": ids, "labels": labels}])
        ours.append((out["loss"], out["grad_norm"], out["lr"]))
    for step, (a, b) in enumerate(zip(ours, ref_traj)):
        assert a[0] == pytest.approx(b[0], rel=2e-4, abs=2e-4), ("loss", step, a, b)
        assert a[1] == pytest.approx(b[1], rel=2e-3, abs=2e-4), ("grad norm", step, a, b)
        assert a[2] == pytest.approx(b[2], rel=1e-6, abs=1e-12), ("lr", step, a, b)
    assert ours[0][2] == 0.0 and ours[-1][0] < ours[0][0]              # first step at lr 0, then the loss moves
    final = t.model.state_dict()
    worst = max((final[k] - ref_final[k]).abs().max().item() for k in ref_final)
    assert worst < 5e-4, worst


@pytest.mark.parametrize("router_overrides", [
    ["--model.moe_router=softmax_topk", "--model.moe_aux_loss_weight=0.01", "--model.moe_router_z_loss_weight=0.001"],
    ["--model.moe_router=sigmoid_topk", "--model.moe_shared_experts=1", "--model.moe_router_z_loss_weight=0.001"],
], ids=["softmax_top2", "sigmoid_bias_balanced"])
def test_moe_steps_match_the_reference(monkeypatch, router_overrides):
    """Mixture-of-experts variant of the same run (4 experts, top-2): routing, auxiliary losses, the sigmoid router's
    bias nudging and moving average follow the reference step by step."""
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    from kempnerforge_b200.config import load_config
    from kempnerforge_b200.training.trainer import Trainer

    overrides = ["--model.num_experts=4", "--model.moe_top_k=2", "--model.n_layers=2", "--train.max_steps=8",
                 *router_overrides]
    batches = _batches(8)
    init: dict = {}
    ref_traj, ref_final = _reference_run(batches, init, overrides)
    cfg = load_config(PRESET, overrides + ["--metrics.log_interval=1000"])
    t = Trainer(cfg, init_dist=False)
    assert set(t.model.state_dict()) == set(init)
    t.model.load_state_dict(init)
    for step, ((ids, labels), want) in enumerate(zip(batches, ref_traj)):
        out = t.train_step([{"input_ids": ids, "labels": labels}])
        t.step += 1
        assert out["loss"] == pytest.approx(want[0], rel=3e-4, abs=3e-4), ("loss", step, out, want)
        assert out["grad_norm"] == pytest.approx(want[1], rel=5e-3, abs=5e-4), ("grad norm", step, out, want)
    final = t.model.state_dict()
    worst = max((final[k].float() - ref_final[k].float()).abs().max().item() for k in ref_final)
    assert worst < 1e-3, worst


@pytest.mark.parametrize("opt_overrides", [
    ["--optimizer.name=muon", "--optimizer.lr=0.02"],
    ["--optimizer.name=lion", "--optimizer.lr=1e-4"],
    ["--optimizer.name=schedule_free_adamw", "--optimizer.lr=1e-3", "--scheduler.name=none",
     "--optimizer.schedule_free_warmup_steps=3"],
], ids=["muon", "lion", "schedule_free"])
def test_other_optimizers_match_the_reference(monkeypatch, opt_overrides):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    from kempnerforge_b200.config import load_config
    from kempnerforge_b200.training.trainer import Trainer

    overrides = ["--model.n_layers=2", "--train.max_steps=6", *opt_overrides]
    batches = _batches(6)
    init: dict = {}
    ref_traj, ref_final = _reference_run(batches, init, overrides)
    cfg = load_config(PRESET, overrides + ["--metrics.log_interval=1000"])
    t = Trainer(cfg, init_dist=False)
    t.model.load_state_dict(init)
    for step, ((ids, labels), want) in enumerate(zip(batches, ref_traj)):
        out = t.train_step([{"input_ids": ids, "labels": labels}])
        t.step += 1
        assert out["loss"] == pytest.approx(want[0], rel=5e-4, abs=5e-4), ("loss", step, out, want)
    final = t.model.state_dict()
    keys = list(ref_final)
    if "muon" in " ".join(opt_overrides):
        # The reference's Muon does not override zero_grad, so `optimizer.zero_grad()` in its training loop never
        # clears the gradients of the parameters its inner AdamW owns (1-D tensors): they accumulate from step to
        # step there.  This framework clears them; the matrices Muon itself updates are compared.
        keys = [k for k in keys if ref_final[k].dim() >= 2]
    worst = max((final[k].float() - ref_final[k].float()).abs().max().item() for k in keys)
    assert worst < 2e-3, worst



# --------------------------------------------------------------------------- two gloo ranks against the reference's FSDP2
def _rank_batches(rank, world, steps):
    """The global batch of 4 sequences split over the ranks, drawn from one stream on every rank."""
    out = []
    for ids, labels in _batches(steps):
        rows = slice(rank * 4 // world, (rank + 1) * 4 // world)
        out.append((ids[rows].contiguous(), labels[rows].contiguous()))
    return out


def _two_rank_worker(rank, world, port, impl, steps, init_file, out_dir, plan="resident"):
    import os
    import traceback

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), CUDA_VISIBLE_DEVICES="")
    torch.set_num_threads(1)
    try:
        # tensor-parallel ranks share the whole batch; data-parallel ranks split it
        batches = _batches(steps) if plan == "tensor_parallel" else _rank_batches(rank, world, steps)
        init = torch.load(init_file)
        traj = []
        if impl == "reference":          # the reference library: fully_shard over a CPU mesh, its own clip / optimizer / schedule
            if str(REF) not in sys.path:
                sys.path.insert(0, str(REF))
            from kempnerforge.config.loader import load_config
            from kempnerforge.distributed.parallel import apply_fsdp2
            from kempnerforge.distributed.utils import clip_grad_norm_
            from kempnerforge.model.transformer import Transformer
            from kempnerforge.training.loss import build_loss_fn
            from kempnerforge.training.optimizer import build_optimizer
            from kempnerforge.training.scheduler import build_scheduler
            from torch.distributed.device_mesh import init_device_mesh
            from torch.distributed.fsdp import MixedPrecisionPolicy

            dist.init_process_group("gloo")
            cfg = load_config(PRESET, [])
            model = Transformer(cfg.model)
            model.load_state_dict(init)
            if plan == "tensor_parallel":
                from kempnerforge.distributed.tensor_parallel import apply_tensor_parallel

                apply_tensor_parallel(model, init_device_mesh("cpu", (world,), mesh_dim_names=("tp",)))
            else:
                mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("dp_shard",))
                apply_fsdp2(model, mesh, mp_policy=MixedPrecisionPolicy(param_dtype=torch.float32, reduce_dtype=torch.float32))
            opt = build_optimizer(model, cfg.optimizer)
            sched = build_scheduler(opt, cfg.scheduler, max_steps=cfg.train.max_steps)
            loss_fn = build_loss_fn(cfg.train)
            for ids, labels in batches:
                loss = loss_fn(model(ids), labels)
                loss.backward()
                norm = clip_grad_norm_(model, cfg.train.grad_clip_norm)
                opt.step()
                sched.step()
                opt.zero_grad()
                mean = loss.detach().clone()
                dist.all_reduce(mean)
                traj.append((float(mean) / world, float(norm)))
            final = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v).detach().clone()
                     for k, v in model.state_dict().items()}
        else:
            from kempnerforge_b200.config import load_config
            from kempnerforge_b200.training.trainer import Trainer

            layout = ([f"--distributed.tp={world}", "--distributed.dp_shard=1"] if plan == "tensor_parallel" else
                      [f"--distributed.dp_shard={world}", f"--distributed.param_sharding={plan}"])
            cfg = load_config(PRESET, layout + ["--metrics.log_interval=1000"])
            t = Trainer(cfg)

            def is_sharded(p):
                return getattr(getattr(p, "_kf_flat", None), "sharded", False)

            assert any(is_sharded(p) for p in t.model.parameters()) == (plan == "sharded")
            def tp_dim(p):
                spec = getattr(p, "_kf_shard", None)
                return spec[1] if spec is not None and spec[0] == "tp" else None

            assert any(tp_dim(p) is not None for p in t.model.parameters()) == (plan == "tensor_parallel")
            for name, p in t.model.named_parameters():     # same starting point as the reference
                if is_sharded(p):
                    t.engine.load_full_parameter(p, init[name])
                elif tp_dim(p) is not None:
                    p.data.copy_(init[name].chunk(world, dim=tp_dim(p))[rank])
                else:
                    p.data.copy_(init[name])
            for ids, labels in batches:
                out = t.train_step([{"input_ids": ids, "labels": labels}])
                mean = torch.tensor(out["loss"], dtype=torch.float64)
                dist.all_reduce(mean)                      # (tensor-parallel ranks report the same loss: mean = itself)
                traj.append((float(mean) / world, out["grad_norm"]))
            final = {}
            for n, p in t.model.named_parameters():
                if is_sharded(p):
                    final[n] = t.engine.full_parameter(p).clone()
                elif tp_dim(p) is not None:
                    parts = [torch.empty_like(p.data) for _ in range(world)]
                    dist.all_gather(parts, p.data.contiguous())
                    final[n] = torch.cat(parts, dim=tp_dim(p))
                else:
                    final[n] = p.detach().clone()
        torch.save((traj, final), os.path.join(out_dir, f"{impl}_{rank}.pt"))
    except Exception:
        with open(os.path.join(out_dir, f"err_{impl}_{rank}.txt"), "w") as fh:
            fh.write(traceback.format_exc())
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("plan", ["resident", "sharded", "tensor_parallel"])
def test_two_gloo_ranks_follow_the_reference_fsdp2_run(tmp_path, plan):
    """The CPU plumbing configuration at world size 2: this package's data-parallel engine, with resident and with
    sharded (ZeRO-3) parameters, against the reference's FSDP2 (``fully_shard`` over a CPU mesh), and this package's
    tensor parallelism against the reference's DTensor plan; same initial weights, same batches."""
    import os
    import socket

    import torch.multiprocessing as mp

    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    from kempnerforge.config.loader import load_config as ref_load
    from kempnerforge.model.transformer import Transformer as RefTransformer

    torch.manual_seed(0)
    init_file = str(tmp_path / "init.pt")
    torch.save(RefTransformer(ref_load(PRESET, []).model).state_dict(), init_file)
    steps, world = 8, 2
    results = {}
    for impl in ("reference", "ours"):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        mp.spawn(_two_rank_worker, args=(world, port, impl, steps, init_file, str(tmp_path), plan), nprocs=world, join=True)
        errs = [open(tmp_path / f).read() for f in sorted(os.listdir(tmp_path)) if f.startswith("err_")]
        assert not errs, "\n".join(errs)
        results[impl] = torch.load(tmp_path / f"{impl}_0.pt")
    (ref_traj, ref_final), (traj, final) = results["reference"], results["ours"]
    for step, (a, b) in enumerate(zip(traj, ref_traj)):
        assert a[0] == pytest.approx(b[0], rel=2e-4, abs=2e-4), ("loss", step, a, b)
        assert a[1] == pytest.approx(b[1], rel=2e-3, abs=2e-4), ("grad norm", step, a, b)
    assert traj[-1][0] < traj[0][0]
    assert set(final) <= set(ref_final) and len(final) == len(ref_final)      # untied model: parameters = state dict
    worst = max((final[k].float() - ref_final[k].float()).abs().max().item() for k in final)
    assert worst < 5e-4, worst


def _pipeline_worker(rank, world, port, impl, steps, init_file, out_dir):
    """Two pipeline stages, two micro-batches per step, clipping switched off (the reference clips each stage by its own
    partial norm, this package by the norm over all stages)."""
    import os
    import traceback

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), CUDA_VISIBLE_DEVICES="")
    torch.set_num_threads(1)
    overrides = ["--train.grad_accum_steps=2", "--train.batch_size=2", "--train.grad_clip_norm=1e9"]
    try:
        init = torch.load(init_file)
        traj = []
        if impl == "reference":
            if str(REF) not in sys.path:
                sys.path.insert(0, str(REF))
            from kempnerforge.config.loader import load_config
            from kempnerforge.distributed.pipeline_parallel import (build_pipeline_schedule, build_pipeline_stage,
                                                                    build_stage_module)
            from kempnerforge.distributed.utils import clip_grad_norm_
            from kempnerforge.training.loss import build_loss_fn
            from kempnerforge.training.optimizer import build_optimizer
            from kempnerforge.training.scheduler import build_scheduler
            from torch.distributed.device_mesh import init_device_mesh

            dist.init_process_group("gloo")
            cfg = load_config(PRESET, overrides)
            mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("pp",))
            device = torch.device("cpu")
            model = build_stage_module(cfg.model, rank, world).to(device=device, dtype=torch.float32)
            model.load_state_dict({k: init[k] for k in model.state_dict()})
            stage = build_pipeline_stage(model, mesh, device, batch_size=2, seq_len=128, param_dtype=torch.float32)
            schedule = build_pipeline_schedule(stage=stage, n_microbatches=2, loss_fn=build_loss_fn(cfg.train), schedule="1f1b")
            opt = build_optimizer(model, cfg.optimizer)
            sched = build_scheduler(opt, cfg.scheduler, max_steps=cfg.train.max_steps)
            for ids, labels in _batches(steps):
                losses: list = []
                if rank == 0:
                    schedule.step(ids, target=labels, losses=losses)
                else:
                    schedule.step(target=labels, losses=losses)
                norm = clip_grad_norm_(model, cfg.train.grad_clip_norm)
                opt.step()
                sched.step()
                opt.zero_grad()
                traj.append((sum(float(x) for x in losses) / max(1, len(losses)), float(norm)))
            final = {k: v.detach().clone() for k, v in model.state_dict().items()}
        else:
            from kempnerforge_b200.config import load_config
            from kempnerforge_b200.training.trainer import Trainer

            cfg = load_config(PRESET, overrides + [f"--distributed.pp={world}", "--distributed.dp_shard=1",
                                                   "--metrics.log_interval=1000"])
            t = Trainer(cfg)
            assert not t.model.load_state_dict(init, strict=False).missing_keys
            for ids, labels in _batches(steps):
                out = t.train_step([{"input_ids": ids[:2], "labels": labels[:2]}, {"input_ids": ids[2:], "labels": labels[2:]}])
                traj.append((out["loss"], out["grad_norm"]))
            final = {k: v.detach().clone() for k, v in t.model.state_dict().items()}
        torch.save((traj, final), os.path.join(out_dir, f"{impl}_{rank}.pt"))
    except Exception:
        with open(os.path.join(out_dir, f"err_{impl}_{rank}.txt"), "w") as fh:
            fh.write(traceback.format_exc())
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_two_pipeline_stages_follow_the_reference_schedule(tmp_path):
    """This package's 1F1B runner against the reference's ``torch.distributed.pipelining`` schedule on two gloo ranks."""
    import os
    import socket

    import torch.multiprocessing as mp

    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    from kempnerforge.config.loader import load_config as ref_load
    from kempnerforge.model.transformer import Transformer as RefTransformer

    torch.manual_seed(0)
    init_file = str(tmp_path / "init.pt")
    torch.save(RefTransformer(ref_load(PRESET, []).model).state_dict(), init_file)
    steps, world = 6, 2
    results = {}
    for impl in ("reference", "ours"):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        mp.spawn(_pipeline_worker, args=(world, port, impl, steps, init_file, str(tmp_path)), nprocs=world, join=True)
        errs = [open(tmp_path / f).read() for f in sorted(os.listdir(tmp_path)) if f.startswith("err_")]
        assert not errs, "\n".join(errs)
        results[impl] = [torch.load(tmp_path / f"{impl}_{r}.pt") for r in range(world)]
    ref, ours = results["reference"], results["ours"]
    for step in range(steps):
        want_loss = ref[world - 1][0][step][0]                                   # the last stage holds the loss
        want_norm = sum(ref[r][0][step][1] ** 2 for r in range(world)) ** 0.5    # its stages report partial norms
        for r in range(world):                                                   # here every stage reports both
            assert ours[r][0][step][0] == pytest.approx(want_loss, rel=2e-4, abs=2e-4), ("loss", step, r)
            assert ours[r][0][step][1] == pytest.approx(want_norm, rel=2e-3, abs=2e-4), ("grad norm", step, r)
    for r in range(world):
        assert set(ours[r][1]) == set(ref[r][1]), r                              # same layer-to-stage assignment and names
        worst = max((ours[r][1][k].float() - ref[r][1][k].float()).abs().max().item() for k in ref[r][1])
        assert worst < 5e-4, (r, worst)
