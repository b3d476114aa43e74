"""Checkpoints are interchangeable with the reference implementation in both directions (single process, CPU):
a checkpoint written by the reference's CheckpointManager loads into this framework's model / optimizer / train state
and gives the same logits, and the other way round.  Skipped when the reference package is not installed under
``baseline/_ref``."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"

pytestmark = pytest.mark.skipif(not (REF / "kempnerforge").is_dir(), reason="reference package not installed")

DENSE = ["--model.dim=64", "--model.n_layers=2", "--model.n_heads=4", "--model.n_kv_heads=2", "--model.vocab_size=128",
         "--model.max_seq_len=32", "--train.seq_len=32", "--train.batch_size=2"]
MOE = DENSE + ["--model.num_experts=4", "--model.moe_top_k=2", "--model.moe_shared_experts=1", "--train.compile_model=false"]


def _reference(overrides, ckpt_dir):
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    from kempnerforge.checkpoint.manager import CheckpointManager
    from kempnerforge.config.loader import load_config
    from kempnerforge.model.transformer import Transformer
    from kempnerforge.training.optimizer import build_optimizer

    cfg = load_config(None, overrides + [f"--checkpoint.dir={ckpt_dir}"])
    model = Transformer(cfg.model)
    opt = build_optimizer(model, cfg.optimizer)
    return cfg, model, opt, CheckpointManager(cfg.checkpoint, model, opt)


def _ours(overrides, ckpt_dir):
    from kempnerforge_b200.checkpoint import CheckpointManager
    from kempnerforge_b200.config import load_config
    from kempnerforge_b200.models.transformer import Transformer
    from kempnerforge_b200.training.optimizer import build_optimizer

    cfg = load_config(None, overrides + [f"--checkpoint.dir={ckpt_dir}"])
    model = Transformer(cfg.model)
    opt = build_optimizer(model, cfg.optimizer)
    return cfg, model, opt, CheckpointManager(cfg.checkpoint, model, opt)


def _one_step(model, opt, ids):
    logits = model(ids)
    torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), ids.reshape(-1)).backward()
    opt.step()
    opt.zero_grad()


def _moments(opt):
    return {k: v["exp_avg"] for k, v in opt.state_dict()["state"].items()}


@pytest.mark.parametrize("overrides", [DENSE, MOE], ids=["dense", "moe"])
def test_reference_checkpoint_loads_here_and_ours_loads_there(tmp_path, overrides, monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    torch.manual_seed(0)
    ids = torch.randint(0, 128, (2, 16))
    # reference -> ours
    _, ref_model, ref_opt, ref_ckpt = _reference(overrides, tmp_path / "ref")
    _one_step(ref_model, ref_opt, ids)
    ref_ckpt.save(step=5, tokens_seen=123)
    assert {".metadata", "metadata.json", "train_state.pt"} <= set(os.listdir(tmp_path / "ref" / "step_5"))
    _, model, opt, ckpt = _ours(overrides, tmp_path / "ref")
    assert set(model.state_dict()) == set(ref_model.state_dict())           # same parameter names
    step, tokens, _ = ckpt.load()
    assert (step, tokens) == (5, 123)
    ref_model.eval(), model.eval()
    with torch.no_grad():
        assert torch.allclose(model(ids), ref_model(ids), atol=1e-5)
    ours_m, ref_m = _moments(opt), _moments(ref_opt)
    assert len(ours_m) == len(ref_m) > 0
    assert all(torch.equal(ours_m[k], ref_m[k]) for k in ref_m)
    # ours -> reference
    model.train()
    _one_step(model, opt, ids)
    _, _, _, ckpt2 = _ours(overrides, tmp_path / "ours")
    ckpt2.model, ckpt2.optimizer = model, opt
    ckpt2.save(step=6, tokens_seen=200)
    ckpt2.wait()
    _, ref_model2, ref_opt2, ref_ckpt2 = _reference(overrides, tmp_path / "ours")
    loaded = ref_ckpt2.load()
    assert tuple(loaded[:2]) == (6, 200)
    ref_model2.eval(), model.eval()
    with torch.no_grad():
        assert torch.allclose(ref_model2(ids), model(ids), atol=1e-5)
    back = _moments(ref_opt2)
    assert all(torch.equal(back[k], v) for k, v in _moments(opt).items())


_REF_FSDP_SAVER = r'''
import os, sys, torch
sys.path.insert(0, sys.argv[2])
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh
from kempnerforge.checkpoint.manager import CheckpointManager
from kempnerforge.config.loader import load_config
from kempnerforge.distributed.parallel import build_parallel_model
from kempnerforge.training.optimizer import build_optimizer
from kempnerforge.training.scheduler import build_scheduler

out = sys.argv[1]
cfg = load_config(None, sys.argv[3:] + ["--train.mixed_precision=fp32", "--train.compile_model=false",
                                        "--distributed.dp_shard=2", f"--checkpoint.dir={out}"])
dist.init_process_group("gloo")
mesh = init_device_mesh("cpu", (2,), mesh_dim_names=("dp_shard",))   # the reference's own set-up needs GPUs
torch.manual_seed(0)
model = build_parallel_model(cfg.model, torch.device("cpu"), mesh, ac_mode="none", param_dtype=torch.float32,
                             compile_model=False, fp8=False)
opt = build_optimizer(model, cfg.optimizer)
sched = build_scheduler(opt, cfg.scheduler, max_steps=100)
torch.manual_seed(1)
ids = torch.randint(0, 128, (2, 16))
logits = model(ids)
torch.nn.functional.cross_entropy(logits.reshape(-1, 128), ids.reshape(-1)).backward()
opt.step(); sched.step(); opt.zero_grad()
CheckpointManager(cfg.checkpoint, model, opt).save(step=7, tokens_seen=77, scheduler=sched)
full = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v).clone() for k, v in model.state_dict().items()}
if dist.get_rank() == 0:
    torch.save(full, os.path.join(out, "weights.pt"))
dist.barrier()
dist.destroy_process_group()
'''

_OURS_LOADER = r'''
import os, sys, torch
sys.path.insert(0, sys.argv[2])
from kempnerforge_b200.config import load_config
from kempnerforge_b200.training.trainer import Trainer

world = int(os.environ.get("WORLD_SIZE", "1"))
extra = [f"--distributed.dp_shard={world}"] if world > 1 else []
cfg = load_config(None, sys.argv[3:] + extra + ["--train.mixed_precision=fp32", f"--checkpoint.dir={sys.argv[1]}",
                                                 "--metrics.log_interval=1000"])
t = Trainer(cfg, init_dist=world > 1)
t.setup_checkpointing()
want = torch.load(os.path.join(sys.argv[1], "weights.pt"))
got = t.model.state_dict()
worst = max((got[k].float() - want[k].float()).abs().max().item() for k in want)
if int(os.environ.get("RANK", "0")) == 0:
    print(f"RESULT step={t.step} tokens={t.tokens_seen} keys={len(want)} worst={worst:.3e}")
'''


@pytest.mark.parametrize("world", [1, 2])
def test_sharded_reference_checkpoint_reshards_into_our_trainer(tmp_path, world):
    """The reference trains with FSDP2 on two gloo ranks and saves DTensor shards; our trainer resumes from that
    checkpoint on one rank and on two (reshard on load), with identical weights."""
    import subprocess

    saver, loader = tmp_path / "ref_saver.py", tmp_path / "ours_loader.py"
    saver.write_text(_REF_FSDP_SAVER)
    loader.write_text(_OURS_LOADER)
    ckpt = tmp_path / "ck"
    ckpt.mkdir()
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    launch = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--master-addr", "127.0.0.1"]
    r = subprocess.run([*launch, "--nproc-per-node=2", "--master-port", "29981", str(saver), str(ckpt), str(REF), *DENSE],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    assert (ckpt / "step_7" / ".metadata").exists() and (ckpt / "step_7" / "__1_0.distcp").exists()
    r2 = subprocess.run([*launch, f"--nproc-per-node={world}", "--master-port", "29982", str(loader), str(ckpt), str(ROOT),
                         *DENSE], capture_output=True, text=True, env=env, timeout=300)
    assert r2.returncode == 0, r2.stdout[-1500:] + r2.stderr[-3000:]
    line = [ln for ln in r2.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    fields = dict(f.split("=") for f in line.split()[1:])
    assert fields["step"] == "7" and fields["tokens"] == "77" and int(fields["keys"]) > 10
    assert float(fields["worst"]) == 0.0


_OURS_SAVER = r'''
import os, sys, torch
sys.path.insert(0, sys.argv[2])
from kempnerforge_b200.config import load_config
from kempnerforge_b200.training.trainer import Trainer

cfg = load_config(None, sys.argv[3:] + ["--distributed.dp_shard=2", "--train.mixed_precision=fp32", "--train.max_steps=100",
                                         f"--checkpoint.dir={sys.argv[1]}", "--metrics.log_interval=1000"])
t = Trainer(cfg)
t.setup_checkpointing()
g = torch.Generator().manual_seed(1 + t.dp_rank)
for _ in range(2):
    tok = torch.randint(0, 128, (2, 33), generator=g)
    t.train_step([{"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}])
    t.step += 1
t.tokens_seen = 256
t.save_checkpoint()
t.ckpt.wait()
if t.rank == 0:
    torch.save({k: v.detach().clone() for k, v in t.model.state_dict().items()}, os.path.join(sys.argv[1], "weights.pt"))
'''

_REF_FSDP_LOADER = r'''
import os, sys, torch
sys.path.insert(0, sys.argv[2])
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh
from kempnerforge.checkpoint.manager import CheckpointManager
from kempnerforge.config.loader import load_config
from kempnerforge.distributed.parallel import build_parallel_model
from kempnerforge.training.optimizer import build_optimizer
from kempnerforge.training.scheduler import build_scheduler

out = sys.argv[1]
cfg = load_config(None, sys.argv[3:] + ["--train.mixed_precision=fp32", "--train.compile_model=false",
                                        "--distributed.dp_shard=2", f"--checkpoint.dir={out}"])
dist.init_process_group("gloo")
mesh = init_device_mesh("cpu", (2,), mesh_dim_names=("dp_shard",))
model = build_parallel_model(cfg.model, torch.device("cpu"), mesh, ac_mode="none", param_dtype=torch.float32,
                             compile_model=False, fp8=False)
opt = build_optimizer(model, cfg.optimizer)
sched = build_scheduler(opt, cfg.scheduler, max_steps=100)
step, tokens, _ = CheckpointManager(cfg.checkpoint, model, opt).load(scheduler=sched)
want = torch.load(os.path.join(out, "weights.pt"))
got = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v) for k, v in model.state_dict().items()}
worst = max((got[k].float() - want[k].float()).abs().max().item() for k in want)
moments = sum(1 for st in opt.state.values() if "exp_avg" in st and float(st["exp_avg"].abs().sum()) > 0)
if dist.get_rank() == 0:
    print(f"RESULT step={step} tokens={tokens} keys={len(want)} worst={worst:.3e} moments={moments}")
dist.barrier()
dist.destroy_process_group()
'''


def test_our_two_rank_checkpoint_loads_into_the_reference_under_fsdp2(tmp_path):
    import subprocess

    saver, loader = tmp_path / "ours_saver.py", tmp_path / "ref_loader.py"
    saver.write_text(_OURS_SAVER)
    loader.write_text(_REF_FSDP_LOADER)
    ckpt = tmp_path / "ck"
    ckpt.mkdir()
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    launch = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1"]
    r = subprocess.run([*launch, "--master-port", "29983", str(saver), str(ckpt), str(ROOT), *DENSE],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    r2 = subprocess.run([*launch, "--master-port", "29984", str(loader), str(ckpt), str(REF), *DENSE],
                        capture_output=True, text=True, env=env, timeout=300)
    assert r2.returncode == 0, r2.stdout[-1500:] + r2.stderr[-3000:]
    line = [ln for ln in r2.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    fields = dict(f.split("=") for f in line.split()[1:])
    assert fields["step"] == "2" and fields["tokens"] == "256" and float(fields["worst"]) == 0.0
    assert int(fields["moments"]) > 10          # optimizer moments arrived too
