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
