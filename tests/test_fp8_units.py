"""FP8 Linear path on CPU (the same arithmetic emulated with torch float8 dtypes): module filter, numerics against
fp32, reuse of quantised weights within a step, configuration rules.  Mirrors tests/unit/test_fp8.py of the reference."""

from __future__ import annotations

import pytest
import torch
from torch import nn

from kempnerforge_b200.config import config_from_dict
from kempnerforge_b200.config.sections import ModelConfig, TrainConfig
from kempnerforge_b200.models.transformer import Transformer
from kempnerforge_b200.ops import fp8
from kempnerforge_b200.ops import functional as F


def test_precision_switch():
    tc = TrainConfig(mixed_precision="fp8")
    assert tc.is_fp8 and tc.param_dtype == torch.bfloat16          # fp8 computes in fp8 but stores bf16
    assert not TrainConfig(mixed_precision="bf16").is_fp8 and TrainConfig(mixed_precision="fp32").param_dtype == torch.float32
    with pytest.raises((ValueError, TypeError)):
        TrainConfig(mixed_precision="int4")


def test_fp8_with_tensor_parallelism_is_rejected_and_with_data_parallelism_accepted():
    base = {"model": dict(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, max_seq_len=32),
            "train": {"mixed_precision": "fp8", "batch_size": 1, "seq_len": 32}}
    with pytest.raises(ValueError):
        config_from_dict({**base, "distributed": {"tp": 2}}).validate(2)
    config_from_dict({**base, "distributed": {"dp_shard": 2}}).validate(2)


def test_convert_model_tags_dense_linears_only():
    torch.manual_seed(0)
    m = Transformer(ModelConfig(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, ffn_hidden_dim=128,
                                max_seq_len=16, num_experts=4, moe_top_k=2, moe_frequency=2, moe_shared_experts=1))
    n = fp8.convert_model(m)
    tagged = {name for name, p in m.named_parameters() if fp8.is_fp8_weight(p)}
    assert n == len(tagged) > 0
    assert all("experts" not in t and "shared_expert" not in t and "router" not in t and "output_head" not in t
               for t in tagged)
    assert "layers.0.attention.q_proj.weight" in tagged and "layers.0.mlp.down_proj.weight" in tagged
    assert all(getattr(blk, "_kf_fp8_block", False) for blk in m.layers.values())
    odd = nn.Sequential(nn.Linear(24, 40))                          # dims that are not multiples of 16 stay bf16
    assert fp8.convert_model(odd) == 0


def _tagged_linear(out_f=32, in_f=64):
    torch.manual_seed(1)
    lin = nn.Linear(in_f, out_f, bias=False).to(torch.bfloat16)
    lin.weight._kf_fp8 = True
    return lin


def test_fp8_linear_tracks_the_fp32_product_forward_and_backward():
    lin = _tagged_linear()
    x = torch.randn(4, 16, 64, dtype=torch.bfloat16, requires_grad=True)
    assert F._fp8_route(x, [lin.weight])
    y = F.linear(x, lin.weight)
    assert y.shape == (4, 16, 32) and y.dtype == torch.bfloat16
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(True), lin.weight.detach().float().requires_grad_(True)
    (xf @ wf.t()).backward(g.float())
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()   # noqa: E731
    assert rel(y, xf.detach() @ wf.detach().t()) < 0.08
    assert rel(x.grad, xf.grad) < 0.15 and rel(lin.weight.grad, wf.grad) < 0.15    # e5m2 gradients are coarse


def test_fused_fp8_linear_splits_weight_gradients():
    a, b = _tagged_linear(32, 64), _tagged_linear(16, 64)
    x = torch.randn(32, 64, dtype=torch.bfloat16, requires_grad=True)
    y = F.fused_linear(x, [a.weight, b.weight])
    assert y.shape == (32, 48)
    y.float().square().sum().backward()
    assert a.weight.grad.shape == (32, 64) and b.weight.grad.shape == (16, 64) and x.grad is not None
    one = F.linear(x.detach(), a.weight)
    assert torch.allclose(one.float(), y[:, :32].detach().float(), atol=0.15, rtol=0.1)   # joint scale vs own scale


def test_quantised_weights_are_reused_until_the_weight_changes(monkeypatch):
    lin = _tagged_linear()
    calls = []
    real = fp8.quantize

    def counting(x2, *a, **k):
        calls.append(tuple(x2.shape))
        return real(x2, *a, **k)

    monkeypatch.setattr(fp8, "quantize", counting)
    x = torch.randn(16, 64, dtype=torch.bfloat16, requires_grad=True)
    for _ in range(3):                                              # micro-batches / recomputation of one step
        F.linear(x, lin.weight).float().sum().backward()
    weight_quantisations = [c for c in calls if c == (32, 64)]
    assert len(weight_quantisations) == 2                           # row-major copy once, transposed copy once
    with torch.no_grad():
        lin.weight.add_(0.01)                                       # what an optimizer step does
    F.linear(x, lin.weight).float().sum().backward()
    assert len([c for c in calls if c == (32, 64)]) == 4


def test_fp8_model_trains_on_cpu():
    torch.manual_seed(2)
    m = Transformer(ModelConfig(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=128,
                                max_seq_len=16)).to(torch.bfloat16)
    fp8.convert_model(m)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    ids = torch.randint(0, 64, (4, 16))
    first = None
    for _ in range(25):
        opt.zero_grad()
        loss = m.compute_loss(ids, ids)
        first = float(loss) if first is None else first
        loss.backward()
        opt.step()
    assert float(loss) < 0.7 * first
