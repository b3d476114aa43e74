"""Token datasets.

``MemoryMappedDataset`` serves fixed-length windows from pre-tokenised ``.npy`` / ``.bin`` shards
without reading them into memory; ``HuggingFaceDataset`` tokenises and packs a text dataset up
front; ``StreamingHuggingFaceDataset`` does the same lazily with rank-strided documents;
``MixtureDataset`` concatenates datasets and tags every sample with its source.

Every sample is ``{"input_ids": t[:-1], "labels": t[1:]}`` over a window of ``seq_len`` tokens
(callers pass ``train.seq_len + 1``).  With ``pack_sequences`` a third entry ``doc_ids`` marks
document membership (the id increases after every EOS token) and labels that would cross a
document boundary are set to -100.

Parity: kempnerforge/data/dataset.py:27-535 (window arithmetic, ``.bin`` dtype rule uint32 when the
file size is a multiple of four else uint16, per-file remainder dropped, files sorted by name,
state dict keys).  Difference: document ids are computed with a vectorised cumulative sum.
"""

from __future__ import annotations

import logging
from pathlib import Path

import numpy as np
import torch
from torch.utils.data import Dataset, IterableDataset

log = logging.getLogger(__name__)


def compute_packed_output(tokens: np.ndarray, eos_token_id: int) -> dict[str, torch.Tensor]:
    """input_ids / labels / doc_ids for one window of ``seq_len + 1`` tokens."""
    tok = torch.from_numpy(np.asarray(tokens).astype(np.int64))
    is_eos = (tok == eos_token_id).long()
    doc = torch.cumsum(is_eos, 0) - is_eos  # the EOS itself still belongs to the document it closes
    inputs, labels = tok[:-1], tok[1:].clone()
    labels[doc[:-1] != doc[1:]] = -100
    return {"input_ids": inputs, "labels": labels, "doc_ids": doc[:-1].contiguous()}


_compute_packed_output = compute_packed_output


class MemoryMappedDataset(Dataset):
    def __init__(self, data_dir: str, seq_len: int, file_pattern: str = "*.npy", pack_sequences: bool = False,
                 eos_token_id: int | None = None) -> None:
        if pack_sequences and eos_token_id is None:
            raise ValueError("eos_token_id is required when pack_sequences=True")
        self.seq_len = seq_len
        self._pack = pack_sequences
        self._eos = eos_token_id
        self._files = sorted(Path(data_dir).glob(file_pattern))
        if not self._files:
            raise FileNotFoundError(f"No files matching {file_pattern!r} in {data_dir}")
        self._mmaps: list[np.ndarray] = []
        bounds = [0]
        total = 0
        try:
            for f in self._files:
                if f.suffix == ".bin":
                    size = f.stat().st_size
                    dt = np.uint32 if size % 4 == 0 else np.uint16
                    arr = np.memmap(str(f), dtype=dt, mode="r", shape=(size // np.dtype(dt).itemsize,))
                else:
                    arr = np.load(str(f), mmap_mode="r")
                self._mmaps.append(arr)
                total += len(arr)
                bounds.append(bounds[-1] + len(arr) // seq_len)
        except Exception:
            self.close()
            raise
        self._bounds = np.asarray(bounds, dtype=np.int64)
        self._epoch = 0
        log.info("MemoryMappedDataset: %d files, %s tokens, %s samples (seq_len=%d)", len(self._files),
                 f"{total:,}", f"{int(self._bounds[-1]):,}", seq_len)

    def __len__(self) -> int:
        return int(self._bounds[-1])

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        if not 0 <= idx < len(self):
            raise IndexError(f"Index {idx} out of range [0, {len(self)})")
        f = int(np.searchsorted(self._bounds, idx, side="right") - 1)
        lo = (idx - int(self._bounds[f])) * self.seq_len
        window = np.asarray(self._mmaps[f][lo : lo + self.seq_len])
        if self._pack:
            return compute_packed_output(window, self._eos)
        tok = torch.from_numpy(window.astype(np.int64))
        return {"input_ids": tok[:-1], "labels": tok[1:]}

    def state_dict(self) -> dict:
        return {"epoch": self._epoch, "total_samples": len(self)}

    def load_state_dict(self, state: dict) -> None:
        self._epoch = state.get("epoch", 0)

    def close(self) -> None:
        for arr in getattr(self, "_mmaps", []):
            mm = getattr(arr, "_mmap", None)
            if mm is not None:
                try:
                    mm.close()
                except (BufferError, ValueError):
                    pass
        self._mmaps = []

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


def _encode_plain(tokenizer, text: str) -> list[int]:
    """Token ids of ``text`` without BOS / EOS or other special tokens (the packer adds EOS itself)."""
    try:
        return list(tokenizer.encode(text, add_special_tokens=False))
    except TypeError:  # minimal tokenizers without the keyword
        return list(tokenizer.encode(text))


def _pack_token_stream(stream, seq_len: int) -> list[np.ndarray]:
    """Cut a stream of token lists into windows of exactly ``seq_len`` tokens (the tail is dropped)."""
    out, buf = [], []
    for toks in stream:
        buf.extend(toks)
        while len(buf) >= seq_len:
            out.append(np.asarray(buf[:seq_len], dtype=np.int64))
            buf = buf[seq_len:]
    return out


class HuggingFaceDataset(Dataset):
    """Eagerly tokenised + packed text dataset (small corpora, tests, quick experiments).

    ``seq_len`` is the training sequence length: documents are tokenised without special tokens, joined with EOS
    (id 0 when the tokenizer has none) and cut into windows of ``seq_len + 1`` tokens, so a sample's ``input_ids``
    and ``labels`` are ``seq_len`` long.  Documents that tokenise to nothing are skipped.
    """

    def __init__(self, dataset_name: str, seq_len: int, tokenizer_path: str, dataset_config: str | None = None,
                 split: str = "train", text_field: str = "text", pack_sequences: bool = False,
                 raw_dataset=None, tokenizer=None) -> None:
        self.seq_len = seq_len
        self._pack = pack_sequences
        self._sample_idx = 0
        if tokenizer is None:
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(tokenizer_path)
        self.tokenizer = tokenizer
        self._eos = tokenizer.eos_token_id or 0
        if raw_dataset is None:
            import datasets

            raw_dataset = datasets.load_dataset(dataset_name, dataset_config, split=split)

        def stream():
            for row in raw_dataset:
                ids = _encode_plain(tokenizer, row[text_field] or "")
                if not ids:
                    continue
                ids.append(self._eos)
                yield ids

        self._samples = _pack_token_stream(stream(), seq_len + 1)
        self._epoch = 0
        log.info("HuggingFaceDataset %s: %d samples of %d tokens", dataset_name, len(self._samples), seq_len)

    def __len__(self) -> int:
        return len(self._samples)

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        window = self._samples[idx]
        if self._pack:
            return compute_packed_output(window, self._eos)
        tok = torch.from_numpy(window)
        return {"input_ids": tok[:-1], "labels": tok[1:]}

    def state_dict(self) -> dict:
        return {"epoch": self._epoch, "sample_idx": self._sample_idx, "total_sequences": len(self._samples)}

    def load_state_dict(self, state: dict) -> None:
        self._epoch = state.get("epoch", 0)
        self._sample_idx = state.get("sample_idx", 0)


class StreamingHuggingFaceDataset(IterableDataset):
    """Lazily tokenised stream; rank r takes documents r, r + world, ...; resumable by this rank's document count.

    ``seq_len`` is the training sequence length (windows of ``seq_len + 1`` tokens, as in ``HuggingFaceDataset``).
    A Hugging Face stream is shuffled through a ``shuffle_buffer_size`` buffer seeded with ``seed + epoch``, so every
    epoch has its own order and a resumed run sees the order of the run it continues.
    Parity: kempnerforge/data/dataset.py:322-468.
    """

    def __init__(self, dataset_name: str, seq_len: int, tokenizer_path: str, dataset_config: str | None = None,
                 split: str = "train", text_field: str = "text", rank: int = 0, world_size: int = 1,
                 pack_sequences: bool = False, raw_stream=None, tokenizer=None, seed: int = 42,
                 shuffle_buffer_size: int = 10000) -> None:
        self.seed, self.shuffle_buffer_size = seed, shuffle_buffer_size
        self.dataset_name, self.dataset_config, self.split = dataset_name, dataset_config, split
        self.seq_len, self.text_field = seq_len, text_field
        self.tokenizer_path = tokenizer_path
        self.rank, self.world_size = rank, world_size
        self._pack = pack_sequences
        self._tokenizer = tokenizer
        self._raw_stream = raw_stream
        self._docs_consumed = 0
        self._skip_rank_docs = 0
        self._epoch = 0

    def _ensure_tokenizer(self):
        if self._tokenizer is None:
            from transformers import AutoTokenizer

            self._tokenizer = AutoTokenizer.from_pretrained(self.tokenizer_path)
        return self._tokenizer

    def _load_stream(self):
        if self._raw_stream is not None:
            return self._raw_stream
        import datasets

        ds = datasets.load_dataset(self.dataset_name, self.dataset_config, split=self.split, streaming=True)
        if self.shuffle_buffer_size > 0:
            ds = ds.shuffle(seed=self.seed + self._epoch, buffer_size=self.shuffle_buffer_size)
        return ds

    def __iter__(self):
        tok = self._ensure_tokenizer()
        eos = tok.eos_token_id or 0
        window_len = self.seq_len + 1
        info = torch.utils.data.get_worker_info()
        n_workers, wid = (info.num_workers, info.id) if info is not None else (1, 0)
        stride = self.world_size * n_workers
        mine = self.rank * n_workers + wid
        buf: list[int] = []
        seen = 0
        for i, row in enumerate(self._load_stream()):
            if i % stride != mine:
                continue
            seen += 1
            if seen <= self._skip_rank_docs:
                continue
            self._docs_consumed = seen
            ids = _encode_plain(tok, row[self.text_field] or "")
            if not ids:
                continue
            buf.extend(ids)
            buf.append(eos)
            while len(buf) >= window_len:
                window = np.asarray(buf[:window_len], dtype=np.int64)
                buf = buf[window_len:]
                if self._pack:
                    yield compute_packed_output(window, eos)
                else:
                    t = torch.from_numpy(window)
                    yield {"input_ids": t[:-1], "labels": t[1:]}
        self._skip_rank_docs = 0
        self._docs_consumed = 0
        self._epoch += 1

    def state_dict(self) -> dict:
        return {"epoch": self._epoch, "rank_docs_consumed": self._docs_consumed}

    def load_state_dict(self, state: dict) -> None:
        self._skip_rank_docs = state.get("rank_docs_consumed", state.get("docs_consumed", 0))
        self._docs_consumed = self._skip_rank_docs
        self._epoch = state.get("epoch", 0)


class MixtureDataset(Dataset):
    """Concatenation of datasets; each sample also carries ``dataset_idx`` for per-source metrics."""

    def __init__(self, datasets: list[Dataset], names: list[str]) -> None:
        if len(datasets) != len(names):
            raise ValueError("datasets and names must have the same length")
        if not datasets:
            raise ValueError("MixtureDataset: At least one dataset is required")
        self._datasets = list(datasets)
        self._names = list(names)
        sizes = [len(d) for d in datasets]
        self._cum = [0]
        for s in sizes:
            self._cum.append(self._cum[-1] + s)

    @property
    def cumulative_sizes(self) -> list[int]:
        return list(self._cum)

    @property
    def dataset_names(self) -> list[str]:
        return list(self._names)

    def __len__(self) -> int:
        return self._cum[-1]

    def __getitem__(self, idx: int) -> dict[str, torch.Tensor]:
        which = int(np.searchsorted(np.asarray(self._cum), idx, side="right") - 1)
        sample = dict(self._datasets[which][idx - self._cum[which]])
        sample["dataset_idx"] = torch.tensor(which, dtype=torch.long)
        return sample

    def state_dict(self) -> dict:
        return {f"dataset_{i}": d.state_dict() for i, d in enumerate(self._datasets) if hasattr(d, "state_dict")}

    def load_state_dict(self, state: dict) -> None:
        legacy = state.get("datasets")          # list form written by earlier checkpoints of this package
        for i, d in enumerate(self._datasets):
            if not hasattr(d, "load_state_dict"):
                continue
            if f"dataset_{i}" in state:
                d.load_state_dict(state[f"dataset_{i}"])
            elif legacy is not None and i < len(legacy):
                d.load_state_dict(legacy[i])
