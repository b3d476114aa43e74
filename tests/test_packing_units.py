"""Sequence packing end to end on CPU: document ids and boundary labels from a token stream, the block-diagonal causal
mask they imply, ignore-index handling in the losses, and the model's isolation of packed documents.

Behaviours of the reference's packing support (kempnerforge/data/dataset.py, kempnerforge/model/attention.py,
kempnerforge/training/loss.py)."""

import numpy as np
import pytest
import torch

from kempnerforge_b200.config import ModelConfig
from kempnerforge_b200.data.dataset import MemoryMappedDataset, compute_packed_output
from kempnerforge_b200.models import Transformer
from kempnerforge_b200.ops import functional as F
from kempnerforge_b200.training import chunked_cross_entropy, cross_entropy

EOS = 7


# --------------------------------------------------------------------------- token stream -> ids and labels
def test_a_stream_without_separator_is_one_document():
    out = compute_packed_output(np.array([1, 2, 3, 4, 5]), EOS)
    assert out["input_ids"].tolist() == [1, 2, 3, 4]
    assert out["labels"].tolist() == [2, 3, 4, 5]
    assert out["doc_ids"].tolist() == [0, 0, 0, 0]


def test_the_separator_belongs_to_the_document_it_ends():
    out = compute_packed_output(np.array([1, 2, EOS, 3, 4]), EOS)
    assert out["doc_ids"].tolist() == [0, 0, 0, 1]
    # the separator is still predicted; the position AFTER it must not predict across the boundary
    assert out["labels"].tolist() == [2, EOS, -100, 4]


def test_three_documents_and_a_trailing_separator():
    out = compute_packed_output(np.array([1, EOS, 2, 3, EOS, 4, EOS]), EOS)
    assert out["doc_ids"].tolist() == [0, 0, 1, 1, 1, 2]
    assert out["labels"].tolist() == [EOS, -100, 3, EOS, -100, EOS]


def test_consecutive_separators_open_empty_documents():
    out = compute_packed_output(np.array([1, EOS, EOS, 2, 3]), EOS)
    assert out["doc_ids"].tolist() == [0, 0, 1, 2]
    assert out["labels"].tolist() == [EOS, -100, -100, 3]


def test_packed_output_types():
    out = compute_packed_output(np.array([1, 2, EOS, 3], dtype=np.uint16), EOS)
    assert out["input_ids"].dtype == torch.long and out["labels"].dtype == torch.long
    assert out["doc_ids"].dtype in (torch.long, torch.int32)
    assert out["input_ids"].shape == out["labels"].shape == out["doc_ids"].shape


# --------------------------------------------------------------------------- the mask the ids imply
def _mask(doc_ids: torch.Tensor) -> torch.Tensor:
    s = doc_ids.shape[-1]
    same = doc_ids.unsqueeze(-1) == doc_ids.unsqueeze(-2)
    return same & torch.tril(torch.ones(s, s, dtype=torch.bool))


def test_one_document_gives_the_causal_mask():
    m = _mask(torch.zeros(6, dtype=torch.long))
    assert torch.equal(m, torch.tril(torch.ones(6, 6, dtype=torch.bool)))


def test_documents_do_not_see_each_other_and_every_token_sees_itself():
    ids = torch.tensor([0, 0, 0, 1, 1, 2])
    m = _mask(ids)
    assert not m[3:5, :3].any() and not m[5, :5].any()
    assert m.diagonal().all()
    assert m[:3, :3].equal(torch.tril(torch.ones(3, 3, dtype=torch.bool)))


# --------------------------------------------------------------------------- losses and the ignore index
def test_cross_entropy_skips_ignored_targets():
    torch.manual_seed(0)
    logits = torch.randn(2, 6, 11)
    labels = torch.randint(0, 11, (2, 6))
    labels[0, 2] = labels[1, 5] = -100
    keep = labels != -100
    want = torch.nn.functional.cross_entropy(logits[keep], labels[keep])
    assert torch.allclose(cross_entropy(logits, labels), want, atol=1e-6)


def test_cross_entropy_with_every_target_ignored_is_zero_not_nan():
    logits = torch.randn(1, 4, 5, requires_grad=True)
    loss = cross_entropy(logits, torch.full((1, 4), -100))
    assert loss.item() == 0.0
    loss.backward()
    assert torch.count_nonzero(logits.grad) == 0


@pytest.mark.parametrize("chunk", [1, 3, 64])
def test_chunked_cross_entropy_matches_the_plain_one_with_ignored_targets(chunk):
    torch.manual_seed(1)
    h = torch.randn(2, 7, 16)
    w = torch.randn(23, 16) * 0.3
    labels = torch.randint(0, 23, (2, 7))
    labels[0, :2] = -100
    logits = h @ w.t()
    want = cross_entropy(logits, labels)
    got = chunked_cross_entropy(logits, labels, chunk_size=chunk)
    assert torch.allclose(got, want, atol=1e-5)
    fused = F.linear_cross_entropy(h, w, labels, chunk_tokens=max(1, chunk))   # head + loss without all logits at once
    assert torch.allclose(fused, want, atol=1e-5)


def test_chunked_cross_entropy_all_ignored():
    logits = torch.randn(1, 5, 9)
    assert chunked_cross_entropy(logits, torch.full((1, 5), -100), chunk_size=2).item() == 0.0


# --------------------------------------------------------------------------- the model
@pytest.fixture(scope="module")
def tiny():
    torch.manual_seed(0)
    cfg = ModelConfig(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=97, max_seq_len=32)
    return Transformer(cfg).eval()


def test_document_ids_keep_the_output_shape_and_none_changes_nothing(tiny):
    tok = torch.randint(0, 97, (2, 12))
    plain = tiny(tok)
    assert tiny(tok, doc_ids=torch.zeros(2, 12, dtype=torch.long)).shape == plain.shape
    assert torch.equal(tiny(tok, doc_ids=None), plain)


def test_a_single_document_equals_plain_causal_attention(tiny):
    tok = torch.randint(0, 97, (1, 10))
    assert torch.allclose(tiny(tok, doc_ids=torch.zeros(1, 10, dtype=torch.long)), tiny(tok), atol=1e-5)


def test_a_document_is_not_affected_by_what_is_packed_before_it(tiny):
    torch.manual_seed(3)
    doc = torch.randint(0, 97, (1, 5))
    a, b = torch.randint(0, 97, (1, 4)), torch.randint(0, 97, (1, 4))
    ids = torch.tensor([[0] * 4 + [1] * 5])
    out_a = tiny(torch.cat([a, doc], dim=1), doc_ids=ids)[:, 4:]
    out_b = tiny(torch.cat([b, doc], dim=1), doc_ids=ids)[:, 4:]
    # rotary positions continue across the packed sequence (as in the reference), so only the prefix CONTENT may not matter
    assert torch.allclose(out_a, out_b, atol=1e-5)
    leaked = tiny(torch.cat([a, doc], dim=1))[:, 4:]
    assert not torch.allclose(leaked, tiny(torch.cat([b, doc], dim=1))[:, 4:], atol=1e-5)


def test_gradients_flow_through_a_packed_batch():
    torch.manual_seed(0)
    cfg = ModelConfig(dim=32, n_layers=1, n_heads=2, n_kv_heads=2, vocab_size=50, max_seq_len=16)
    model = Transformer(cfg)
    tok = torch.randint(0, 50, (2, 9))
    ids = torch.tensor([[0, 0, 0, 1, 1, 1, 2, 2], [0] * 8])
    labels = tok[:, 1:].clone()
    labels[0, 2] = labels[0, 5] = -100
    loss = cross_entropy(model(tok[:, :-1], doc_ids=ids), labels)
    loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


# --------------------------------------------------------------------------- the memory-mapped dataset
@pytest.fixture()
def packed_dir(tmp_path):
    stream = np.array([1, 2, EOS, 3, 4, 5, EOS, 6, 1, 2, 3, EOS, 4, 5, 6, 1, 2], dtype=np.uint16)
    np.save(tmp_path / "shard.npy", stream)
    return str(tmp_path)


def test_packed_windows_carry_document_ids_and_masked_boundaries(packed_dir):
    ds = MemoryMappedDataset(packed_dir, 8, pack_sequences=True, eos_token_id=EOS)
    item = ds[0]
    assert set(item) >= {"input_ids", "labels", "doc_ids"}
    # a window holds seq_len tokens: seq_len - 1 inputs and their shifted targets
    assert item["input_ids"].tolist() == [1, 2, EOS, 3, 4, 5, EOS]
    assert item["doc_ids"].tolist() == [0, 0, 0, 1, 1, 1, 1]
    assert item["labels"].tolist() == [2, EOS, -100, 4, 5, EOS, -100]
    ds.close()


def test_windows_without_packing_have_no_document_ids(packed_dir):
    ds = MemoryMappedDataset(packed_dir, 8)
    assert "doc_ids" not in ds[0] and ds[0]["labels"].tolist() == [2, EOS, 3, 4, 5, EOS, 6]
    ds.close()


def test_packing_without_a_separator_id_is_rejected(packed_dir):
    with pytest.raises(ValueError):
        MemoryMappedDataset(packed_dir, 8, pack_sequences=True)


def test_pack_sequences_is_off_by_default_and_configurable():
    from kempnerforge_b200.config import config_from_dict

    assert config_from_dict({}).data.pack_sequences is False
    assert config_from_dict({"data": {"pack_sequences": True}}).data.pack_sequences is True
