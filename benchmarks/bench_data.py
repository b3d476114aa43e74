"""Host-side data path: memory-mapped reads, packed sequences, the stateful loader, mixtures.
Parity: benchmarks/bench_data.py:14-123 in the reference."""

from __future__ import annotations

import atexit
import shutil
import tempfile
from pathlib import Path

import numpy as np
import torch

from benchmarks.runner import Case, print_results, run_suite

SUITE = "data"


def _make_shards(n_files: int = 4, n_tokens: int = 100_000) -> Path:
    root = Path(tempfile.mkdtemp(prefix="kf_bench_data_"))
    atexit.register(shutil.rmtree, root, ignore_errors=True)
    rng = np.random.default_rng(0)
    for i in range(n_files):
        tok = rng.integers(0, 32000, size=n_tokens, dtype=np.uint16)
        tok[rng.integers(0, n_tokens, size=n_tokens // 300)] = 2  # sprinkle EOS for the packed case
        np.save(root / f"shard_{i}.npy", tok)
    return root


def cases(device: torch.device):
    from kempnerforge_b200.data.dataloader import StatefulDataLoader
    from kempnerforge_b200.data.dataset import MemoryMappedDataset, MixtureDataset
    from kempnerforge_b200.data.sampler import DistributedSampler

    root = _make_shards()
    seq = 513
    plain = MemoryMappedDataset(str(root), seq)
    packed = MemoryMappedDataset(str(root), seq, pack_sequences=True, eos_token_id=2)
    n = min(len(plain), 500)

    def read_all(ds):
        def fn():
            for i in range(n):
                ds[i]
        return fn

    yield Case(f"MemoryMappedDataset ({n} samples)", read_all(plain), tokens_per_iter=n * seq, host_timed=True)
    yield Case(f"MemoryMappedDataset packed, doc_ids ({n} samples)", read_all(packed), tokens_per_iter=n * seq,
               host_timed=True)

    def loader_epoch():
        sampler = DistributedSampler(plain, num_replicas=1, rank=0, shuffle=True, seed=0)
        loader = StatefulDataLoader(plain, batch_size=8, sampler=sampler, num_workers=0)
        for k, _batch in enumerate(loader):
            if k >= 40:
                break

    yield Case("StatefulDataLoader (40 batches of 8, no workers)", loader_epoch, tokens_per_iter=40 * 8 * seq,
               host_timed=True)

    mix = MixtureDataset([plain, packed], ["plain", "packed"])

    def mix_read():
        step = max(len(mix) // n, 1)
        for i in range(0, step * n, step):
            mix[i]

    yield Case(f"MixtureDataset ({n} samples over 2 sources)", mix_read, tokens_per_iter=n * seq, host_timed=True)


if __name__ == "__main__":
    print_results(run_suite(SUITE, torch.device("cpu")), "data")
