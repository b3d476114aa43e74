"""Decoding, loss functions, evaluation loop and pipeline-stage construction on CPU.

Mirrors tests/unit/test_generate.py, test_loss.py, test_eval.py and test_pipeline_parallel.py of the reference."""

from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as TF

from kempnerforge_b200.config.sections import EvalConfig, ModelConfig, TrainConfig
from kempnerforge_b200.models.attention import KVCache
from kempnerforge_b200.models.generate import generate, sample
from kempnerforge_b200.models.transformer import Transformer
from kempnerforge_b200.parallel.pipeline_parallel import (build_stage_module, compute_layer_assignment,
                                                         schedule_order)
from kempnerforge_b200.training.eval import run_eval, should_build_eval_dataloader
from kempnerforge_b200.training.loss import build_loss_fn, chunked_cross_entropy, cross_entropy, z_loss


def _cfg(**kw):
    base = dict(dim=32, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=50, ffn_hidden_dim=64, max_seq_len=24)
    base.update(kw)
    return ModelConfig(**base)


def _model(**kw):
    torch.manual_seed(0)
    return Transformer(_cfg(**kw))


# --------------------------------------------------------------------------- KV cache / sampling / generation
def test_kv_cache_updates_incrementally_and_overflows_loudly():
    c = KVCache(2, 8, 2, 4, torch.float32, "cpu")
    assert c.seq_len == 0 and c.k.shape == (2, 8, 2, 4)
    k, v = c.update(torch.ones(2, 3, 2, 4), torch.ones(2, 3, 2, 4) * 2)
    assert k.shape == (2, 3, 2, 4) and c.seq_len == 3 and float(v.sum()) == 2 * 3 * 2 * 4 * 2
    k, _ = c.update(torch.zeros(2, 1, 2, 4), torch.zeros(2, 1, 2, 4))
    assert k.shape[1] == 4 and float(k[:, :3].sum()) == 2 * 3 * 2 * 4
    with pytest.raises(ValueError):
        c.update(torch.zeros(2, 5, 2, 4), torch.zeros(2, 5, 2, 4))
    c.reset()
    assert c.seq_len == 0


def test_sampling_rules():
    logits = torch.tensor([[0.0, 1.0, 5.0, 2.0], [3.0, 0.0, 0.0, 0.0]])
    assert sample(logits, temperature=0.0).tolist() == [2, 0]
    g = torch.Generator().manual_seed(0)
    draws = torch.cat([sample(logits[:1], 1.0, top_k=2, generator=g) for _ in range(200)])
    assert set(draws.flatten().tolist()) <= {2, 3}
    draws = torch.cat([sample(logits[:1], 1.0, top_p=0.5, generator=g) for _ in range(100)])
    assert set(draws.flatten().tolist()) == {2}      # the first token already covers more than half the mass
    hot = torch.cat([sample(logits[:1], 100.0, generator=g) for _ in range(400)])
    assert len(set(hot.flatten().tolist())) == 4       # a high temperature flattens the distribution
    cold = torch.cat([sample(logits[:1], 0.05, generator=g) for _ in range(100)])
    assert set(cold.flatten().tolist()) == {2}
    assert sample(logits, 1.0, generator=g).shape == (2,)


def test_generate_contract():
    m = _model()
    m.train()
    prompt = torch.randint(0, 50, (2, 5))
    out = generate(m, prompt, max_new_tokens=6, temperature=0.0)
    assert out.shape == (2, 11) and torch.equal(out[:, :5], prompt) and m.training
    assert int(out.min()) >= 0 and int(out.max()) < 50
    assert torch.equal(generate(m, prompt, 6, temperature=0.0), out)              # greedy is deterministic
    assert all(p.grad is None for p in m.parameters())
    m.eval()
    generate(m, prompt, 2, temperature=0.0)
    assert not m.training                                                          # an eval model stays in eval
    assert torch.equal(generate(m, prompt, 0), prompt)
    with pytest.raises(ValueError, match="exceeds model max_seq_len"):                 # never silently clipped
        generate(m, prompt, 1000, temperature=0.0)


def test_generate_stops_at_eos_and_pads_finished_rows():
    m = _model()
    prompt = torch.randint(0, 50, (2, 4))
    free = generate(m, prompt, 8, temperature=0.0)
    eos = int(free[0, 5])   # the second token row 0 emits
    out = generate(m, prompt, 8, temperature=0.0, eos_token_id=eos)
    row = out[0, 4:].tolist()
    first = row.index(eos)
    assert all(t == eos for t in row[first:])
    assert out.shape[1] <= 12


def test_incremental_decoding_matches_the_full_forward_with_grouped_kv():
    m = _model(n_kv_heads=1).eval()
    ids = torch.randint(0, 50, (1, 9))
    full = m(ids)
    caches = [KVCache(1, 16, 1, m.config.head_dim, torch.float32, "cpu") for _ in m.layers]
    steps = [m(ids[:, :4], kv_caches=caches)] + [m(ids[:, i:i + 1], kv_caches=caches) for i in range(4, 9)]
    assert torch.allclose(torch.cat(steps, dim=1), full, atol=1e-4)


# --------------------------------------------------------------------------- losses
def test_cross_entropy_matches_torch_and_ignores_minus_100():
    torch.manual_seed(1)
    logits = torch.randn(3, 7, 11, requires_grad=True)
    labels = torch.randint(0, 11, (3, 7))
    labels[0, :3] = -100
    want = TF.cross_entropy(logits.reshape(-1, 11), labels.reshape(-1), ignore_index=-100)
    got = cross_entropy(logits, labels)
    assert got.shape == () and torch.allclose(got, want, atol=1e-6)
    got.backward()
    g = logits.grad.clone()
    logits.grad = None
    want.backward()
    assert torch.allclose(g, logits.grad, atol=1e-6) and float(g[0, :3].abs().sum()) == 0.0
    assert float(cross_entropy(logits, torch.full_like(labels, -100))) == 0.0
    perfect = torch.full((1, 4, 11), -30.0)
    perfect[0, torch.arange(4), torch.arange(4)] = 30.0
    assert float(cross_entropy(perfect, torch.arange(4)[None])) < 1e-6


@pytest.mark.parametrize("chunk", [1, 4, 5, 21, 4096])
def test_chunked_cross_entropy_equals_the_plain_loss(chunk):
    torch.manual_seed(2)
    logits = torch.randn(3, 7, 11, requires_grad=True)
    labels = torch.randint(0, 11, (3, 7))
    labels[1, 2:5] = -100
    a = chunked_cross_entropy(logits, labels, chunk_size=chunk)
    b = cross_entropy(logits, labels)
    assert torch.allclose(a, b, atol=1e-6)
    (ga,) = torch.autograd.grad(a, logits)
    (gb,) = torch.autograd.grad(b, logits)
    assert torch.allclose(ga, gb, atol=1e-6)
    assert float(chunked_cross_entropy(logits, torch.full_like(labels, -100), chunk)) == 0.0


def test_z_loss_scales_with_weight_and_logit_magnitude():
    logits = torch.randn(2, 5, 11, requires_grad=True)
    assert float(z_loss(logits, 0.0)) == 0.0
    small, large = z_loss(logits * 0.01, 1e-4), z_loss(logits * 100.0, 1e-4)
    assert 0 < float(small) < float(large)
    want = 1e-4 * torch.logsumexp(logits, -1).pow(2).mean()
    assert torch.allclose(z_loss(logits, 1e-4), want)
    z_loss(logits, 1e-2).backward()
    assert logits.grad.abs().sum() > 0


def test_build_loss_fn_composition():
    logits, labels = torch.randn(2, 5, 11), torch.randint(0, 11, (2, 5))
    base = cross_entropy(logits, labels)
    assert torch.equal(build_loss_fn(TrainConfig())(logits, labels), base)
    chunked = build_loss_fn(TrainConfig(loss_fn="chunked_cross_entropy", ce_chunk_size=3))(logits, labels)
    assert torch.allclose(chunked, base, atol=1e-6)
    default_chunk = build_loss_fn(TrainConfig(loss_fn="chunked_cross_entropy"))(logits, labels)
    assert torch.allclose(default_chunk, base, atol=1e-6)
    with_z = build_loss_fn(TrainConfig(z_loss_weight=1e-2))(logits, labels)
    assert torch.allclose(with_z, base + z_loss(logits, 1e-2))


# --------------------------------------------------------------------------- evaluation
class _Batches:
    def __init__(self, n, bs=2, s=8, vocab=50):
        g = torch.Generator().manual_seed(3)
        self.items = [{"input_ids": torch.randint(0, vocab, (bs, s), generator=g),
                       "labels": torch.randint(0, vocab, (bs, s), generator=g)} for _ in range(n)]

    def __iter__(self):
        return iter(self.items)


def test_run_eval_reports_loss_and_perplexity_and_restores_the_mode():
    m = _model()
    m.train()
    cfg = SimpleNamespace(eval=EvalConfig(enabled=True, steps=5))
    out = run_eval(m, _Batches(2), cfg, torch.device("cpu"))       # 2 batches, 5 steps: the loader wraps around
    assert set(out) == {"eval/loss", "eval/perplexity"} and m.training
    assert out["eval/perplexity"] == pytest.approx(math.exp(out["eval/loss"]))
    assert abs(out["eval/loss"] - math.log(50)) < 1.0               # random init: close to uniform
    assert all(p.grad is None for p in m.parameters())
    m.eval()
    run_eval(m, _Batches(1), cfg, torch.device("cpu"))
    assert not m.training
    one = run_eval(m, _Batches(1), SimpleNamespace(eval=EvalConfig(enabled=True, steps=1)), torch.device("cpu"))
    b = _Batches(1).items[0]
    assert one["eval/loss"] == pytest.approx(float(m.compute_loss(b["input_ids"], b["labels"])), rel=1e-5)


def test_eval_loader_is_built_only_for_text_runs_with_a_source():
    mk = lambda **kw: SimpleNamespace(eval=EvalConfig(**kw), is_vlm=False)  # noqa: E731
    assert should_build_eval_dataloader(mk(enabled=True, dataset_path="/data/val"))
    assert should_build_eval_dataloader(mk(enabled=True, hf_dataset_name="org/ds"))
    assert not should_build_eval_dataloader(mk(enabled=True))
    assert not should_build_eval_dataloader(mk(enabled=False, dataset_path="/data/val"))
    vlm = SimpleNamespace(eval=EvalConfig(enabled=True, dataset_path="/data/val"), is_vlm=True)
    assert not should_build_eval_dataloader(vlm)
    with pytest.raises(ValueError):
        EvalConfig(steps=0)


# --------------------------------------------------------------------------- pipeline stages
@pytest.mark.parametrize("n,pp,want", [(8, 4, [2, 2, 2, 2]), (10, 4, [3, 3, 2, 2]), (5, 1, [5]), (4, 4, [1, 1, 1, 1]),
                                       (7, 2, [4, 3])])
def test_layer_assignment(n, pp, want):
    out = compute_layer_assignment(n, pp)
    assert [end - start for start, end in out] == want
    assert [i for start, end in out for i in range(start, end)] == list(range(n))


def test_layer_assignment_rejects_too_many_stages():
    with pytest.raises(ValueError):
        compute_layer_assignment(2, 4)
    with pytest.raises(ValueError):
        compute_layer_assignment(2, 0)


def test_stage_modules_partition_the_model_and_chain_to_the_same_output():
    cfg = _cfg(n_layers=5)
    torch.manual_seed(0)
    full = Transformer(cfg)
    stages = [build_stage_module(cfg, r, 3) for r in range(3)]
    assert [sorted(s.layers.keys(), key=int) for s in stages] == [["0", "1"], ["2", "3"], ["4"]]
    first, mid, last = stages
    assert first.token_embedding is not None and first.output_head is None and first.norm is None
    assert mid.token_embedding is None and mid.output_head is None
    assert last.token_embedding is None and last.output_head is not None and last.norm is not None
    sd = full.state_dict()
    total = 0
    for s in stages:
        own = s.state_dict()
        assert set(own) <= set(sd)                       # stage keys are the global names
        s.load_state_dict({k: sd[k] for k in own})
        total += sum(p.numel() for p in s.parameters())
    assert total == sum(p.numel() for p in full.parameters())
    ids = torch.randint(0, 50, (2, 6))
    h = first(ids)
    assert h.shape == (2, 6, 32)
    h = last(mid(h))
    logits = h @ last.output_head.proj.weight.t()
    assert torch.allclose(logits, full(ids), atol=1e-4)
    labels = torch.randint(0, 50, (2, 6))
    assert torch.allclose(last.stage_loss(h, labels), full.compute_loss(ids, labels), atol=1e-5)
    solo = build_stage_module(cfg, 0, 1)
    assert solo.token_embedding is not None and solo.output_head is not None and len(solo.layers) == 5


@pytest.mark.parametrize("kind", ["1f1b", "gpipe"])
@pytest.mark.parametrize("stages,micro", [(2, 4), (4, 8), (4, 2), (3, 1)])
def test_schedule_order_runs_every_micro_batch_forward_then_backward(kind, stages, micro):
    for stage in range(stages):
        order = schedule_order(kind, stage, stages, micro)
        assert len(order) == 2 * micro
        for i in range(micro):
            assert order.index(("F", i)) < order.index(("B", i))
        assert [i for op, i in order if op == "F"] == list(range(micro))
        assert [i for op, i in order if op == "B"] == list(range(micro))
        if kind == "1f1b":
            in_flight = peak = 0
            for op, _ in order:
                in_flight += 1 if op == "F" else -1
                peak = max(peak, in_flight)
            assert peak <= min(micro, stages - stage)       # bounded activation memory
    with pytest.raises(ValueError):
        schedule_order("interleaved_1f1b", 0, stages, micro)
