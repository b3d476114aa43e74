"""Datasets, packing, samplers and the resumable loader."""

import numpy as np
import pytest
import torch

from kempnerforge_b200.data import (
    DistributedSampler,
    MemoryMappedDataset,
    MixtureDataset,
    MixtureSampler,
    StatefulDataLoader,
    compute_packed_output,
)


@pytest.fixture
def shards(tmp_path):
    rng = np.random.default_rng(0)
    for i, n in enumerate((100, 57)):
        np.save(tmp_path / f"shard_{i}.npy", rng.integers(0, 1000, n).astype(np.uint16))
    return tmp_path


def test_mmap_windows_and_shift(shards):
    ds = MemoryMappedDataset(str(shards), seq_len=9)
    assert len(ds) == 100 // 9 + 57 // 9
    a = np.load(shards / "shard_0.npy")
    s = ds[3]
    assert torch.equal(s["input_ids"], torch.from_numpy(a[27:35].astype(np.int64)))
    assert torch.equal(s["labels"], torch.from_numpy(a[28:36].astype(np.int64)))
    b = np.load(shards / "shard_1.npy")
    first_of_second = ds[100 // 9]
    assert torch.equal(first_of_second["input_ids"], torch.from_numpy(b[0:8].astype(np.int64)))
    with pytest.raises(IndexError):
        ds[len(ds)]
    with pytest.raises(FileNotFoundError):
        MemoryMappedDataset(str(shards), 9, file_pattern="*.bin")
    ds.close()


def test_bin_dtype_rule(tmp_path):
    np.arange(10, dtype=np.uint32).tofile(tmp_path / "a.bin")  # 40 bytes -> uint32
    ds = MemoryMappedDataset(str(tmp_path), 5, file_pattern="*.bin")
    assert ds[1]["input_ids"].tolist() == [5, 6, 7, 8]
    ds.close()
    np.arange(9, dtype=np.uint16).tofile(tmp_path / "b.bin")  # 18 bytes -> uint16
    ds = MemoryMappedDataset(str(tmp_path), 3, file_pattern="b.bin")
    assert len(ds) == 3 and ds[2]["labels"].tolist() == [7, 8]
    ds.close()


def test_packing_doc_ids_and_boundary_labels():
    eos = 9
    tokens = np.array([1, 2, eos, 3, 4, eos, 5, 6])
    out = compute_packed_output(tokens, eos)
    assert out["doc_ids"].tolist() == [0, 0, 0, 1, 1, 1, 2]
    assert out["labels"].tolist() == [2, eos, -100, 4, eos, -100, 6]
    with pytest.raises(ValueError):
        MemoryMappedDataset("/tmp", 4, pack_sequences=True)


def test_distributed_sampler_partition_and_resume():
    samplers = [DistributedSampler(103, num_replicas=4, rank=r, seed=5) for r in range(4)]
    parts = [list(s) for s in samplers]
    assert all(len(p) == 25 for p in parts)
    flat = sum(parts, [])
    assert len(set(flat)) == 100  # disjoint, drop_last
    again = list(DistributedSampler(103, 4, 1, seed=5))
    assert again == parts[1]
    s = DistributedSampler(103, 4, 1, seed=5)
    s.set_skip(7)
    assert list(s) == parts[1][7:]
    s.set_epoch(1)
    assert list(s) != parts[1]
    assert s.state_dict()["epoch"] == 1


def test_mixture_sampler_quotas_and_update():
    cum = [0, 100, 300]
    ms = MixtureSampler(cum, [3.0, 1.0], num_replicas=2, rank=0, seed=1)
    idx = list(ms)
    assert len(idx) == 150
    n0 = sum(i < 100 for i in idx)
    assert n0 == round(0.75 * 150)  # dataset 0 is oversampled by wrapping
    assert list(MixtureSampler(cum, [3.0, 1.0], 2, 0, seed=1)) == idx
    ms.update_weights([0.0, 1.0])
    assert all(i >= 100 for i in ms)
    hot = MixtureSampler(cum, [3.0, 1.0], 2, 0, seed=1, temperature=100.0)
    assert abs(sum(i < 100 for i in hot) - 75) <= 2  # high temperature -> nearly uniform
    with pytest.raises(ValueError):
        MixtureSampler(cum, [0.0, 0.0])
    with pytest.raises(ValueError):
        MixtureSampler(cum, [1.0, -1.0])


def test_mixture_dataset_tags_source(shards):
    a = MemoryMappedDataset(str(shards), 9, "shard_0.npy")
    b = MemoryMappedDataset(str(shards), 9, "shard_1.npy")
    mix = MixtureDataset([a, b], ["a", "b"])
    assert len(mix) == len(a) + len(b) and mix.dataset_names == ["a", "b"]
    assert mix[0]["dataset_idx"].item() == 0 and mix[len(a)]["dataset_idx"].item() == 1
    with pytest.raises(ValueError):
        MixtureDataset([a], ["a", "b"])


def test_stateful_loader_exact_resume_and_epoch_roll(shards):
    def make():
        ds = MemoryMappedDataset(str(shards), 5)
        return StatefulDataLoader(ds, 4, DistributedSampler(len(ds), 1, 0, seed=3), num_workers=0)

    ref = make()
    it = iter(ref)
    batches = [next(it)["input_ids"] for _ in range(5)]
    half = make()
    it2 = iter(half)
    for _ in range(2):
        next(it2)
    state = half.state_dict()
    resumed = make()
    resumed.load_state_dict(state)
    it3 = iter(resumed)
    for k in range(2, 5):
        assert torch.equal(next(it3)["input_ids"], batches[k])
    # a second resume from the resumed loader still lines up
    state2 = resumed.state_dict()
    again = make()
    again.load_state_dict(state2)
    assert again.state_dict()["batches_yielded"] == 5
    # epoch roll-over
    full = make()
    n = 0
    for _ in full:
        n += 1
    assert n == len(full) and full.state_dict()["epoch"] == 1 and full.state_dict()["batches_yielded"] == 0


def test_synthetic_tokens_resume():
    from kempnerforge_b200.training.trainer import SyntheticTokens

    a = SyntheticTokens(100, 2, 8, seed=1, dp_rank=0)
    next(a)
    state = a.state_dict()
    want = next(a)
    b = SyntheticTokens(100, 2, 8, seed=1, dp_rank=0)
    b.load_state_dict(state)
    got = next(b)
    assert torch.equal(got["input_ids"], want["input_ids"])
    assert torch.equal(want["labels"][:, :-1], want["input_ids"][:, 1:])
    other = next(SyntheticTokens(100, 2, 8, seed=1, dp_rank=1))
    assert not torch.equal(other["input_ids"], next(SyntheticTokens(100, 2, 8, seed=1, dp_rank=0))["input_ids"])
