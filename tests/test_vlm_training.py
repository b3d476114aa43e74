"""Vision-language training through the Trainer on CPU: every architecture takes optimizer steps, the frozen
encoder stays frozen, a freeze-schedule boundary changes the trainable set and keeps optimizer moments."""

import pytest
import torch
from PIL import Image

from kempnerforge_b200.config import config_from_dict
from kempnerforge_b200.data import build_vlm_dataloader
from kempnerforge_b200.data.vlm_dataset import HuggingFaceVLMDataset
from kempnerforge_b200.training.trainer import Trainer
from tests.test_vlm_data import ToyTokenizer


def _cfg(arch="joint_decoder", **vlm_extra):
    vlm = dict(arch=arch, max_text_len=12, **vlm_extra)
    return config_from_dict({
        "model": dict(dim=64, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=128, ffn_hidden_dim=128, max_seq_len=64),
        "train": dict(batch_size=2, seq_len=16, max_steps=6, mixed_precision="fp32", seed=0),
        "optimizer": dict(lr=1e-2), "scheduler": dict(name="constant", warmup_steps=0),
        "vision_encoder": dict(type="random", feature_dim=32, num_tokens=4),
        "adapter": dict(type="mlp_2layer"),
        "vlm": vlm,
        "metrics": dict(log_interval=100),
    })


def _loader(cfg, n=8):
    tok = ToyTokenizer()
    rows = [{"image": Image.new("RGB", (8, 8), color=(i * 20 % 255, 10, 200)), "text": f"w{i} w{i + 1} w{i + 2} end"}
            for i in range(n)]
    for r in rows:      # the toy vocabulary grows in encounter order: fix it, so two loaders tokenise alike
        tok(r["text"])
    ds = HuggingFaceVLMDataset("toy", "train", "image", "text", "", cfg.vlm.max_text_len, image_size=8, rows=rows,
                               tokenizer=tok)
    return build_vlm_dataloader(cfg, dataset=ds, tokenizer=tok)


@pytest.mark.parametrize("arch", ["joint_decoder", "cross_attention", "mot"])
def test_vlm_trainer_steps(arch):
    extra = {"cross_attention_every_n_layers": 2} if arch == "cross_attention" else {}
    cfg = _cfg(arch, **extra)
    t = Trainer(cfg, init_dist=False, dataloader=_loader(cfg))
    enc_before = [p.detach().clone() for p in t.model.vision_encoder.parameters()]
    losses = [t.train_step()["loss"] for _ in range(5)]
    assert all(l == l and l > 0 for l in losses)
    assert losses[-1] < losses[0]
    for a, b in zip(enc_before, t.model.vision_encoder.parameters()):
        assert torch.equal(a, b) and not b.requires_grad


def test_freeze_schedule_transition_keeps_moments():
    cfg = _cfg("joint_decoder",
               freeze=[{"module": "vision_encoder", "frozen": True}, {"module": "transformer", "frozen": True}],
               freeze_schedule=[{"start_step": 2, "specs": [{"module": "transformer", "frozen": False}]}])
    t = Trainer(cfg, init_dist=False, dataloader=_loader(cfg))
    trainable0 = {n for n, p in t.model.named_parameters() if p.requires_grad}
    assert trainable0 and all(n.startswith("adapter.") for n in trainable0)
    w0 = t.model.transformer.layers["0"].mlp.down_proj.weight.detach().clone()
    for _ in range(2):
        t._maybe_advance_freeze_stage()
        t.train_step()
        t.step += 1
    assert torch.equal(w0, t.model.transformer.layers["0"].mlp.down_proj.weight)      # frozen so far
    adapter_p = next(p for n, p in t.model.named_parameters() if n.startswith("adapter."))
    from kempnerforge_b200.checkpoint.manager import optimizer_state_dict

    before = optimizer_state_dict(t.model, t.optimizer)["state"]
    key = next(k for k in before if k.startswith("adapter."))
    m_before = before[key]["exp_avg"].clone()
    t._maybe_advance_freeze_stage()                                                   # step 2: transformer thaws
    trainable1 = {n for n, p in t.model.named_parameters() if p.requires_grad}
    assert any(n.startswith("transformer.") for n in trainable1) and trainable0 < trainable1
    after = optimizer_state_dict(t.model, t.optimizer)["state"]
    assert torch.allclose(after[key]["exp_avg"].float(), m_before.float())            # moments carried over
    t.train_step()
    assert not torch.equal(w0, t.model.transformer.layers["0"].mlp.down_proj.weight)  # now it trains
    assert adapter_p.requires_grad


def test_vlm_run_reports_the_text_tokens_of_logged_steps():
    cfg = _cfg()
    loader = _loader(cfg)
    t = Trainer(cfg, init_dist=False, dataloader=loader)
    first = next(iter(_loader(cfg)))
    expected = int((first["labels"][:, 1:] != -100).sum())
    assert 0 < expected < first["labels"].numel()
    t.train_step()                                  # the step that becomes step 1 is a logged step
    assert t._text_token_metrics() == {"data/text_tokens_trained": float(expected)}
    t.step = 1
    t.train_step()                                  # step 2 with log_interval=100: nothing is counted
    assert t._text_token_metrics() == {}


def test_resume_after_a_freeze_stage_boundary_is_bit_exact(tmp_path):
    """A checkpoint written after the transformer thawed carries moments for parameters that are frozen at step 0.
    The resuming trainer has to move to the saved step's freeze stage before loading; it then continues exactly
    like the run that never stopped, and the checkpoint's metadata records the freeze set-up."""
    import json

    def make():
        cfg = _cfg("joint_decoder",
                   freeze=[{"module": "vision_encoder", "frozen": True}, {"module": "transformer", "frozen": True}],
                   freeze_schedule=[{"start_step": 2, "specs": [{"module": "transformer", "frozen": False}]}])
        cfg.checkpoint.dir = str(tmp_path / "ckpt")
        cfg.checkpoint.async_mode = "disabled"
        return cfg

    def run(t, n):
        out = []
        for _ in range(n):
            t._maybe_advance_freeze_stage()
            out.append(t.train_step()["loss"])
            t.step += 1
        return out

    cfg = make()
    a = Trainer(cfg, init_dist=False, dataloader=_loader(cfg, n=16))
    a.setup_checkpointing()
    run(a, 3)                                           # steps 0, 1 frozen; step 2 trains the transformer
    a.save_checkpoint()
    a.ckpt.wait()
    meta = json.loads((tmp_path / "ckpt" / "step_3" / "metadata.json").read_text())
    assert {"module": "transformer", "frozen": False} in meta["vlm_freeze"]
    tail_a = run(a, 2)

    cfg_b = make()
    b = Trainer(cfg_b, init_dist=False, dataloader=_loader(cfg_b, n=16))
    assert not any(n.startswith("transformer.") for n, p in b.model.named_parameters() if p.requires_grad)
    b.setup_checkpointing()
    assert b.step == 3
    assert any(n.startswith("transformer.") for n, p in b.model.named_parameters() if p.requires_grad)
    tail_b = run(b, 2)
    assert tail_a == tail_b
    for (n1, p1), (n2, p2) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2), n1
