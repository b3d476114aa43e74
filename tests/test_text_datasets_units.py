"""Memory-mapped shards, the distributed sampler, the stateful loader and the Hugging Face text datasets (with an
in-memory corpus and a toy tokenizer; no network).  Mirrors tests/unit/test_data.py of the reference."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from kempnerforge_b200.data.dataloader import StatefulDataLoader
from kempnerforge_b200.data.dataset import HuggingFaceDataset, MemoryMappedDataset, StreamingHuggingFaceDataset
from kempnerforge_b200.data.sampler import DistributedSampler


class _Tok:
    """Whitespace tokenizer: word i of the vocabulary list -> id i + 1; id 0 ends a document."""

    eos_token_id = 0

    def encode(self, text):
        return [int(w[1:]) + 1 for w in text.split()]


def _docs(n, words):
    return [{"text": " ".join(f"w{(i * 7 + j) % 50}" for j in range(words))} for i in range(n)]


# --------------------------------------------------------------------------- memory-mapped shards
@pytest.fixture
def shard_dir(tmp_path):
    np.save(tmp_path / "a.npy", np.arange(0, 100, dtype=np.uint16))
    np.save(tmp_path / "b.npy", np.arange(1000, 1070, dtype=np.uint16))
    return tmp_path


def test_mmap_windows_lengths_and_boundaries(shard_dir):
    ds = MemoryMappedDataset(str(shard_dir), seq_len=33)
    assert len(ds) == 100 // 33 + 70 // 33 == 5                     # partial windows are dropped per file
    s = ds[0]
    assert s["input_ids"].shape == s["labels"].shape == (32,) and s["input_ids"].dtype == torch.int64
    assert torch.equal(s["labels"][:-1], s["input_ids"][1:])         # labels are the inputs shifted by one
    assert int(ds[2]["input_ids"][0]) == 66 and int(ds[3]["input_ids"][0]) == 1000   # windows never span files
    for bad in (-1, 5):                                              # negative indices are rejected, like the reference
        with pytest.raises(IndexError):
            ds[bad]
    other = MemoryMappedDataset(str(shard_dir), seq_len=10)
    assert len(other) == 17
    ds.load_state_dict({"epoch": 3})
    assert ds.state_dict() == {"epoch": 3, "total_samples": len(ds)}
    with pytest.raises(FileNotFoundError):
        MemoryMappedDataset(str(shard_dir), seq_len=8, file_pattern="*.tokens")
    with pytest.raises(ValueError):
        MemoryMappedDataset(str(shard_dir), seq_len=8, pack_sequences=True)      # packing needs an EOS id


# --------------------------------------------------------------------------- sampler
def test_distributed_sampler_partitions_without_overlap():
    parts = [list(DistributedSampler(103, 4, r, shuffle=True, seed=5, drop_last=True)) for r in range(4)]
    assert all(len(p) == 25 for p in parts)
    flat = [i for p in parts for i in p]
    assert len(set(flat)) == 100 and all(0 <= i < 103 for i in flat)
    padded = [list(DistributedSampler(103, 4, r, shuffle=False, seed=5, drop_last=False)) for r in range(4)]
    assert all(len(p) == 26 for p in padded) and set(i for p in padded for i in p) == set(range(103))


def test_distributed_sampler_determinism_epochs_skip_and_state():
    a = DistributedSampler(50, 2, 0, shuffle=True, seed=1)
    b = DistributedSampler(50, 2, 0, shuffle=True, seed=1)
    first = list(a)
    assert first == list(b) and list(a) == first
    a.set_epoch(1)
    assert list(a) != first and sorted(list(a)) != []
    a.set_epoch(0)
    a.set_skip(7)
    assert list(a) == first[7:]
    a.set_epoch(4)
    state = a.state_dict()
    c = DistributedSampler(50, 2, 0, shuffle=True, seed=99)
    c.load_state_dict(state)
    assert list(c) == list(a)
    assert list(DistributedSampler(10, 1, 0, shuffle=False)) == list(range(10))


# --------------------------------------------------------------------------- loader
def test_stateful_loader_iterates_counts_and_rolls_epochs(shard_dir):
    ds = MemoryMappedDataset(str(shard_dir), seq_len=10)             # 17 samples
    loader = StatefulDataLoader(ds, 4, DistributedSampler(len(ds), 1, 0, shuffle=True, seed=0), 0, False, None, True)
    batches = list(loader)
    assert len(batches) == 4 and batches[0]["input_ids"].shape == (4, 9)
    state = loader.state_dict()
    assert state["epoch"] >= 1 or state.get("batches", 0) == 0
    again = list(loader)
    assert len(again) == 4
    assert not all(torch.equal(x["input_ids"], y["input_ids"]) for x, y in zip(batches, again))   # new epoch, new order


# --------------------------------------------------------------------------- Hugging Face datasets on an in-memory corpus
def test_hf_dataset_packs_documents_into_fixed_windows():
    docs = _docs(20, 9) + [{"text": ""}, {"text": "   "}]            # empty documents are skipped
    ds = HuggingFaceDataset("toy", 15, "", raw_dataset=docs, tokenizer=_Tok())          # windows of 15 + 1 tokens
    assert len(ds) == (20 * 10) // 16
    s = ds[0]
    assert s["input_ids"].shape == s["labels"].shape == (15,) and torch.equal(s["labels"][:-1], s["input_ids"][1:])
    stream = torch.cat([torch.cat([ds[i]["input_ids"], ds[i]["labels"][-1:]]) for i in range(len(ds))])
    assert int((stream == 0).sum()) >= 12                           # document ends (EOS) are inside the stream
    assert ds.state_dict() == {"epoch": 0, "sample_idx": 0, "total_sequences": len(ds)}
    ds.load_state_dict({"epoch": 2, "sample_idx": 5})
    assert ds.state_dict()["epoch"] == 2 and ds.state_dict()["sample_idx"] == 5


def test_hf_dataset_packed_output_carries_document_ids():
    ds = HuggingFaceDataset("toy", 15, "", raw_dataset=_docs(10, 5), tokenizer=_Tok(), pack_sequences=True)
    s = ds[0]
    assert {"input_ids", "labels", "doc_ids"} <= set(s)
    assert s["doc_ids"].shape == s["input_ids"].shape and int(s["doc_ids"].max()) >= 1
    boundary = (s["doc_ids"][1:] != s["doc_ids"][:-1]).nonzero().flatten()
    assert len(boundary) and all(int(s["labels"][int(b)]) == -100 for b in boundary)   # no loss across documents


def test_streaming_dataset_shards_by_document_and_resumes():
    docs = _docs(40, 7)
    full = list(StreamingHuggingFaceDataset("toy", 7, "", raw_stream=docs, tokenizer=_Tok()))
    assert len(full) == (40 * 8) // 8 and full[0]["input_ids"].shape == (7,)
    r0 = list(StreamingHuggingFaceDataset("toy", 7, "", raw_stream=docs, tokenizer=_Tok(), rank=0, world_size=2))
    r1 = list(StreamingHuggingFaceDataset("toy", 7, "", raw_stream=docs, tokenizer=_Tok(), rank=1, world_size=2))
    assert len(r0) == len(r1) == 20
    assert not any(torch.equal(a["input_ids"], b["input_ids"]) for a, b in zip(r0, r1))
    with_empty = [{"text": ""}] + docs
    assert len(list(StreamingHuggingFaceDataset("toy", 7, "", raw_stream=with_empty, tokenizer=_Tok()))) == 40
    ds = StreamingHuggingFaceDataset("toy", 7, "", raw_stream=docs, tokenizer=_Tok())
    it = iter(ds)
    head = [next(it) for _ in range(10)]
    state = ds.state_dict()
    assert state == {"epoch": 0, "rank_docs_consumed": 10}
    resumed = StreamingHuggingFaceDataset("toy", 7, "", raw_stream=docs, tokenizer=_Tok())
    resumed.load_state_dict(state)
    tail = list(resumed)
    assert len(head) + len(tail) == len(full)
    assert torch.equal(tail[0]["input_ids"], full[10]["input_ids"])
    packed = next(iter(StreamingHuggingFaceDataset("toy", 15, "", raw_stream=docs, tokenizer=_Tok(), pack_sequences=True)))
    assert "doc_ids" in packed
