"""Sampling rules and the generation loop on CPU, one behaviour per test.

Behaviours of kempnerforge/model/generate.py (sample: temperature -> top-k -> top-p -> multinomial; generate: prefill
+ one token per step against per-layer KV caches)."""

import pytest
import torch

from kempnerforge_b200.config import ModelConfig
from kempnerforge_b200.models import Transformer
from kempnerforge_b200.models.attention import KVCache
from kempnerforge_b200.models.generate import generate, sample


@pytest.fixture(scope="module")
def model():
    torch.manual_seed(0)
    return Transformer(ModelConfig(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=53, max_seq_len=48))


# --------------------------------------------------------------------------- KV cache
def test_cache_starts_empty_and_has_one_slot_per_kv_head():
    c = KVCache(2, 16, 2, 8, torch.float32, torch.device("cpu"))
    assert c.seq_len == 0 and c.k.shape == (2, 16, 2, 8) and c.v.shape == c.k.shape


def test_cache_update_returns_everything_written_so_far():
    c = KVCache(1, 8, 2, 4, torch.float32, torch.device("cpu"))
    k1, v1 = torch.randn(1, 3, 2, 4), torch.randn(1, 3, 2, 4)
    k, v = c.update(k1, v1)
    assert k.shape == (1, 3, 2, 4) and torch.equal(k, k1) and c.seq_len == 3
    k2, v2 = torch.randn(1, 1, 2, 4), torch.randn(1, 1, 2, 4)
    k, v = c.update(k2, v2)
    assert k.shape == (1, 4, 2, 4) and torch.equal(k[:, :3], k1) and torch.equal(v[:, 3:], v2) and c.seq_len == 4


# --------------------------------------------------------------------------- sample
def test_temperature_zero_is_argmax_and_deterministic():
    logits = torch.tensor([[0.1, 2.0, -1.0], [3.0, 0.0, 0.5]])
    assert sample(logits, temperature=0.0).tolist() == [1, 0]
    assert torch.equal(sample(logits, temperature=0.0), sample(logits, temperature=0.0))


def test_top_k_never_leaves_the_k_largest_logits():
    torch.manual_seed(0)
    logits = torch.randn(1, 40)
    allowed = set(torch.topk(logits, 5, dim=-1).indices[0].tolist())
    drawn = {int(sample(logits, temperature=1.5, top_k=5)) for _ in range(200)}
    assert drawn <= allowed and len(drawn) > 1


def test_top_p_keeps_the_smallest_prefix_that_reaches_the_mass():
    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]]))
    drawn = {int(sample(logits, top_p=0.7)) for _ in range(300)}
    assert drawn == {0, 1}                      # 0.5 alone is below 0.7, 0.5 + 0.3 crosses it
    assert {int(sample(logits, top_p=0.4)) for _ in range(50)} == {0}   # the first token is always kept


def test_low_temperature_concentrates_and_high_temperature_spreads():
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]])
    g = torch.Generator().manual_seed(1)
    cold = [int(sample(logits, temperature=0.1, generator=g)) for _ in range(200)]
    hot = [int(sample(logits, temperature=5.0, generator=g)) for _ in range(200)]
    assert cold.count(0) > 190 and len(set(hot)) == 4 and hot.count(0) < 120


def test_sampling_is_per_row_and_reproducible_with_a_generator():
    logits = torch.tensor([[10.0, 0.0, 0.0], [0.0, 0.0, 10.0]])
    out = sample(logits, temperature=0.5, generator=torch.Generator().manual_seed(3))
    assert out.shape == (2,) and out.tolist() == [0, 2]
    wide = torch.randn(4, 30)
    a = sample(wide, generator=torch.Generator().manual_seed(7))
    b = sample(wide, generator=torch.Generator().manual_seed(7))
    assert torch.equal(a, b)


# --------------------------------------------------------------------------- generate
def test_output_is_the_prompt_followed_by_valid_new_tokens(model):
    prompt = torch.randint(0, 53, (2, 5))
    out = generate(model, prompt, max_new_tokens=7, temperature=0.8, generator=torch.Generator().manual_seed(0))
    assert out.shape == (2, 12) and torch.equal(out[:, :5], prompt)
    assert int(out.min()) >= 0 and int(out.max()) < 53


def test_greedy_generation_repeats_itself_and_matches_the_full_forward(model):
    prompt = torch.randint(0, 53, (1, 4))
    a = generate(model, prompt, max_new_tokens=6, temperature=0.0)
    assert torch.equal(a, generate(model, prompt, max_new_tokens=6, temperature=0.0))
    model.eval()
    seq = prompt
    for _ in range(6):   # the same tokens without any cache
        seq = torch.cat([seq, model(seq)[:, -1].argmax(-1, keepdim=True)], dim=1)
    assert torch.equal(a, seq)


def test_rows_that_hit_eos_are_padded_with_it_and_the_loop_ends_early(model):
    prompt = torch.randint(0, 53, (2, 3))
    first = generate(model, prompt, max_new_tokens=1, temperature=0.0)[:, -1]
    eos = int(first[0])
    out = generate(model, prompt, max_new_tokens=10, temperature=0.0, eos_token_id=eos)
    row = out[0, 3:]
    assert int(row[0]) == eos and bool((row == eos).all())        # finished rows only ever emit the separator again
    if int(first[1]) == eos:
        assert out.shape[1] == 4                                   # every row finished at once: one new token only


def test_training_mode_is_restored_and_eval_mode_is_left_alone(model):
    prompt = torch.randint(0, 53, (1, 3))
    model.train()
    generate(model, prompt, max_new_tokens=2, temperature=0.0)
    assert model.training
    model.eval()
    generate(model, prompt, max_new_tokens=2, temperature=0.0)
    assert not model.training


def test_generation_builds_no_graph(model):
    out = generate(model.train(), torch.randint(0, 53, (1, 3)), max_new_tokens=3)
    assert not out.requires_grad and all(p.grad is None for p in model.parameters())


def test_zero_new_tokens_returns_the_prompt_and_overlong_requests_are_rejected(model):
    prompt = torch.randint(0, 53, (1, 6))
    assert torch.equal(generate(model, prompt, max_new_tokens=0), prompt)
    with pytest.raises(ValueError, match="max_seq_len"):
        generate(model, prompt, max_new_tokens=43)
