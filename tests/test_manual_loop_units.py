"""Hand-written training loops over the library pieces (``build_parallel_model`` + ``build_optimizer`` +
``loss.backward(); clip_grad_norm_(); optimizer.step(); optimizer.zero_grad()``) must train exactly like the
``Trainer``, without any call into the data-parallel engine: with FSDP2 in the reference such a loop is complete
(tests/integration/test_train_step.py, test_vlm_train_step.py), and code ported from it is written that way."""

import os
import socket
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

MODEL = dict(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, max_seq_len=32)


def _job(opt_name, world=1, clip=1.0, dtype="fp32"):
    from kempnerforge_b200.config import config_from_dict

    return config_from_dict({
        "model": MODEL,
        "train": {"batch_size": 2, "seq_len": 16, "max_steps": 10, "mixed_precision": dtype, "seed": 0, "grad_clip_norm": clip},
        "optimizer": {"name": opt_name, "lr": 1e-2 if opt_name == "adamw" else 1e-3},
        "scheduler": {"name": "constant", "warmup_steps": 0},
        "distributed": {"dp_shard": world} if world > 1 else {},
        "metrics": {"log_interval": 1000},
    })


def _batches(n, seed=3):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        tok = torch.randint(0, 128, (2, 17), generator=g)
        out.append({"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()})
    return out


def _manual_run(cfg, init, batches, mesh=None):
    """What a user writes against the reference's API: no engine call anywhere."""
    from kempnerforge_b200.distributed import build_parallel_model, clip_grad_norm_
    from kempnerforge_b200.training.loss import build_loss_fn
    from kempnerforge_b200.training.optimizer import build_optimizer

    model = build_parallel_model(cfg.model, torch.device("cpu"), mesh, param_dtype=cfg.train.param_dtype)
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(init[n])
    opt = build_optimizer(model, cfg.optimizer)
    loss_fn = build_loss_fn(cfg.train)
    traj = []
    for b in batches:
        loss = loss_fn(model(b["input_ids"]), b["labels"])
        loss.backward()
        norm = clip_grad_norm_(model, cfg.train.grad_clip_norm)
        opt.step()
        opt.zero_grad()
        traj.append((float(loss.detach()), float(norm)))
    return traj, {n: p.detach().clone() for n, p in model.named_parameters()}


def _trainer_run(cfg, init, batches, init_dist=False):
    from kempnerforge_b200.training.trainer import Trainer

    t = Trainer(cfg, init_dist=init_dist) if not init_dist else Trainer(cfg)
    with torch.no_grad():
        for n, p in t.model.named_parameters():
            p.copy_(init[n])
    traj = []
    for b in batches:
        out = t.train_step([b])
        traj.append((out["loss"], out["grad_norm"]))
    return traj, {n: p.detach().clone() for n, p in t.model.named_parameters()}, t


def _init_weights():
    from kempnerforge_b200.config import ModelConfig
    from kempnerforge_b200.models import Transformer

    torch.manual_seed(0)
    return {n: p.detach().clone() for n, p in Transformer(ModelConfig(**MODEL)).named_parameters()}


@pytest.mark.parametrize("opt_name", ["adamw", "lion", "muon"])
def test_a_plain_loop_trains_like_the_trainer(opt_name):
    cfg, init, batches = _job(opt_name), _init_weights(), _batches(4)
    want_traj, want_params, _ = _trainer_run(cfg, init, batches)
    got_traj, got_params = _manual_run(cfg, init, batches)
    for step, (a, b) in enumerate(zip(got_traj, want_traj)):
        assert a[0] == pytest.approx(b[0], rel=1e-6), ("loss", step)
        assert a[1] == pytest.approx(b[1], rel=1e-5), ("grad norm", step)
    assert got_traj[-1][0] != got_traj[0][0]
    for n in want_params:
        assert torch.allclose(got_params[n], want_params[n], atol=1e-7), n
        assert not torch.equal(got_params[n], init[n]) or want_params[n].numel() == 0, n     # every parameter moved


def test_clipping_is_applied_once_and_only_to_the_step_it_was_computed_for():
    """A loop that clips in step 1 and not in step 2: the second update must use the unscaled gradient."""
    from kempnerforge_b200.distributed import build_parallel_model, clip_grad_norm_
    from kempnerforge_b200.training.loss import build_loss_fn
    from kempnerforge_b200.training.optimizer import build_optimizer

    for opt_name in ("adamw", "lion"):
        cfg, init, (b1, b2) = _job(opt_name, clip=0.05), _init_weights(), _batches(2)
        model = build_parallel_model(cfg.model, torch.device("cpu"), None, param_dtype=torch.float32)
        with torch.no_grad():
            for n, p in model.named_parameters():
                p.copy_(init[n])
        opt = build_optimizer(model, cfg.optimizer)
        loss_fn = build_loss_fn(cfg.train)
        loss_fn(model(b1["input_ids"]), b1["labels"]).backward()
        assert float(clip_grad_norm_(model, 0.05)) > 0.05
        opt.step()
        opt.zero_grad()
        engine = model._kf_engine
        assert float(engine.grad_scale) == 1.0 and not engine._scale_pending, opt_name
        loss_fn(model(b2["input_ids"]), b2["labels"]).backward()
        opt.step()                                   # no clipping this time
        opt.zero_grad()
        assert all(p.grad is None for p in model.parameters())


def test_zero_grad_after_a_backward_without_a_step_forgets_the_gradients():
    """The loop of a skipped step (non-finite loss): backward, no step, zero_grad.  The next step must not see them."""
    from kempnerforge_b200.distributed import build_parallel_model
    from kempnerforge_b200.training.loss import build_loss_fn
    from kempnerforge_b200.training.optimizer import build_optimizer

    cfg, init, (b1, b2) = _job("adamw"), _init_weights(), _batches(2)
    runs = []
    for skip_first in (True, False):
        model = build_parallel_model(cfg.model, torch.device("cpu"), None, param_dtype=torch.float32)
        with torch.no_grad():
            for n, p in model.named_parameters():
                p.copy_(init[n])
        opt = build_optimizer(model, cfg.optimizer)
        loss_fn = build_loss_fn(cfg.train)
        if skip_first:
            (1e3 * loss_fn(model(b1["input_ids"]), b1["labels"])).backward()
            opt.zero_grad()
        loss_fn(model(b2["input_ids"]), b2["labels"]).backward()
        opt.step()
        runs.append({n: p.detach().clone() for n, p in model.named_parameters()})
    for n in runs[0]:
        assert torch.equal(runs[0][n], runs[1][n]), n


# --------------------------------------------------------------------------- two gloo ranks
def _rank_entry(rank, world, port, out_dir, opt_name):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), CUDA_VISIBLE_DEVICES="")
    torch.set_num_threads(1)
    try:
        from kempnerforge_b200.parallel.setup import init_distributed

        cfg, init = _job(opt_name, world), _init_weights()
        mine = _batches(3 * world)[rank::world]
        want_traj, want_params, t = _trainer_run(cfg, init, mine, init_dist=True)
        mesh = init_distributed(cfg.distributed, seed=0)
        got_traj, got_params = _manual_run(cfg, init, mine, mesh)
        torch.save((want_traj, want_params, got_traj, got_params), os.path.join(out_dir, f"r{rank}.pt"))
    except Exception:
        with open(os.path.join(out_dir, f"err{rank}.txt"), "w") as fh:
            fh.write(traceback.format_exc())
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("opt_name", ["adamw", "lion"])
def test_a_plain_loop_on_two_ranks_trains_like_the_trainer(opt_name):
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_entry, args=(world, port, d, opt_name), nprocs=world, join=True)
        errs = [open(os.path.join(d, f)).read() for f in sorted(os.listdir(d)) if f.startswith("err")]
        assert not errs, "\n".join(errs)
        results = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(world)]
    for want_traj, want_params, got_traj, got_params in results:
        for step, (a, b) in enumerate(zip(got_traj, want_traj)):
            assert a[0] == pytest.approx(b[0], rel=1e-6), ("loss", step)
            assert a[1] == pytest.approx(b[1], rel=1e-5), ("grad norm", step)
        for n in want_params:
            assert torch.allclose(got_params[n], want_params[n], atol=1e-7), n
    for n in results[0][3]:                                   # and the ranks agree with each other
        assert torch.equal(results[0][3][n], results[1][3][n]), n


def test_gradients_written_into_the_flat_buffers_show_up_as_grad_after_backward():
    """On a GPU the fused nodes hand ``None`` to autograd and write weight gradients into the flat buffer; the engine's
    end-of-backward callback must then present those slots as ``.grad``.  Here the deposit is imitated on the CPU."""
    from kempnerforge_b200.distributed import build_parallel_model

    cfg = _job("adamw")
    model = build_parallel_model(cfg.model, torch.device("cpu"), None, param_dtype=torch.float32)
    engine = model._kf_engine
    b = _batches(1)[0]
    model(b["input_ids"]).float().mean().backward()      # the block hooks queue the callback during this pass
    assert not engine._expose_queued and all(p.grad is not None for p in model.parameters())
    name, p = next((n, q) for n, q in model.named_parameters() if n.endswith("q_proj.weight"))
    other = next(q for n, q in model.named_parameters() if n.endswith("k_proj.weight"))
    kept = other.grad
    p.grad = None                                         # what a fused node leaves behind: no autograd gradient,
    p._kf_grad.fill_(2.0)                                 # the value in the flat slot,
    p._kf_grad_live = True                                # and the slot marked as written
    engine._expose_flat_grads()
    assert p.grad is not None and p.grad.data_ptr() == p._kf_grad.data_ptr() and float(p.grad.mean()) == 2.0, name
    assert other.grad is kept                             # gradients that autograd produced are left alone
    model._kf_engine.zero_grad()
    assert all(q.grad is None for q in model.parameters()) and not p._kf_grad_live


def test_a_trainable_parameter_no_node_reached_shows_a_zero_gradient():
    """The flat optimizer update treats a parameter without a gradient as a zero gradient (weight decay still applies);
    ``.grad`` says the same instead of staying ``None``."""
    from torch import nn

    from kempnerforge_b200.config import ModelConfig
    from kempnerforge_b200.models import Transformer
    from kempnerforge_b200.parallel.parallel import apply_fsdp2

    model = Transformer(ModelConfig(**MODEL))
    model.unused = nn.Parameter(torch.ones(8))           # takes no part in the forward pass
    apply_fsdp2(model, None)
    b = _batches(1)[0]
    model(b["input_ids"]).float().mean().backward()
    assert model.unused.grad is not None and float(model.unused.grad.abs().max()) == 0.0
    assert float(model.layers["0"].attention.q_proj.weight.grad.abs().max()) > 0.0
    with torch.no_grad():                                # no graph, no hook, nothing queued
        model(b["input_ids"])
    assert not model._kf_engine._expose_queued


def _hand_built_optimizer_entry(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), CUDA_VISIBLE_DEVICES="")
    torch.set_num_threads(1)
    try:
        from kempnerforge_b200.distributed import build_parallel_model
        from kempnerforge_b200.parallel.setup import init_distributed
        from kempnerforge_b200.training.loss import build_loss_fn

        cfg, init = _job("adamw", world), _init_weights()
        mesh = init_distributed(cfg.distributed, seed=0)
        model = build_parallel_model(cfg.model, torch.device("cpu"), mesh, param_dtype=torch.float32)
        with torch.no_grad():
            for n, p in model.named_parameters():
                p.copy_(init[n])
        opt = torch.optim.SGD(model.parameters(), lr=0.1)       # not from build_optimizer
        model._kf_engine.bind_optimizer(opt)
        loss_fn = build_loss_fn(cfg.train)
        for b in _batches(2 * world)[rank::world]:              # every rank sees different data
            loss_fn(model(b["input_ids"]), b["labels"]).backward()
            opt.step()
            opt.zero_grad()
        torch.save({n: p.detach().clone() for n, p in model.named_parameters()}, os.path.join(out_dir, f"r{rank}.pt"))
    except Exception:
        with open(os.path.join(out_dir, f"err{rank}.txt"), "w") as fh:
            fh.write(traceback.format_exc())
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_a_hand_built_optimizer_bound_to_the_engine_keeps_the_ranks_in_step():
    """A whole-parameter optimizer needs the whole averaged gradient on every rank, not only the local shard of the
    reduce-scatter: after two steps on different data the ranks must hold identical, changed weights."""
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_hand_built_optimizer_entry, args=(world, port, d), nprocs=world, join=True)
        errs = [open(os.path.join(d, f)).read() for f in sorted(os.listdir(d)) if f.startswith("err")]
        assert not errs, "\n".join(errs)
        a, b = (torch.load(os.path.join(d, f"r{r}.pt")) for r in range(world))
    init = _init_weights()
    for n in a:
        assert torch.equal(a[n], b[n]), n
        assert not torch.equal(a[n], init[n]), n
