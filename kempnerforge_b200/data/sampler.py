"""Deterministic, resumable samplers.

``DistributedSampler``: permutation seeded by (seed + epoch), truncated to a multiple of the
replica count, rank r takes positions r, r + R, ...; ``set_skip`` drops already-consumed samples on
resume.  ``MixtureSampler``: per-dataset quotas from (temperature-scaled) weights, every dataset
permuted and rank-strided independently, wrapped around when its quota exceeds its size, then one
global shuffle — all driven by a single generator seeded with (seed + epoch).

Parity: kempnerforge/data/sampler.py:18-348 (index arithmetic, rounding repair in favour of the
largest weights, state dict keys, ``update_weights`` for training phases).
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch.utils.data import Sampler


def _validate_weights(weights: list[float], context: str) -> None:
    if not weights:
        raise ValueError(f"{context}: weights must not be empty")
    if any((not math.isfinite(w)) or w < 0 for w in weights):
        raise ValueError(f"{context}: weights must be finite and non-negative, got {weights}")
    if sum(weights) <= 0:
        raise ValueError(f"{context}: weights must sum to > 0 (at least one positive weight)")


def _replica_info(num_replicas, rank):
    if num_replicas is None:
        num_replicas = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    if rank is None:
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if not 0 <= rank < num_replicas:
        raise ValueError(f"rank {rank} out of range for {num_replicas} replicas")
    return num_replicas, rank


class DistributedSampler(Sampler[int]):
    def __init__(self, dataset_size=None, num_replicas: int | None = None, rank: int | None = None,
                 shuffle: bool = True, seed: int = 0, drop_last: bool = True, *, dataset=None) -> None:
        """The first argument is a sample count or a sized dataset (also accepted as ``dataset=``)."""
        if dataset_size is None:
            if dataset is None:
                raise TypeError("DistributedSampler needs a dataset or its size")
            dataset_size = dataset
        self.dataset_size = dataset_size if isinstance(dataset_size, int) else len(dataset_size)
        self.num_replicas, self.rank = _replica_info(num_replicas, rank)
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        if drop_last:
            self.num_samples = self.dataset_size // self.num_replicas
        else:
            self.num_samples = math.ceil(self.dataset_size / self.num_replicas)
        self.total_size = self.num_samples * self.num_replicas
        self._epoch = 0
        self._skip = 0

    def set_epoch(self, epoch: int) -> None:
        self._epoch = epoch

    def set_skip(self, skip: int) -> None:
        self._skip = max(0, skip)

    def __iter__(self):
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self._epoch)
            order = torch.randperm(self.dataset_size, generator=g).tolist()
        else:
            order = list(range(self.dataset_size))
        if self.drop_last:
            order = order[: self.total_size]
        elif len(order) < self.total_size:
            order += order[: self.total_size - len(order)]
        mine = order[self.rank : self.total_size : self.num_replicas]
        if self._skip:
            mine = mine[self._skip :]
            self._skip = 0
        return iter(mine)

    def __len__(self) -> int:
        return self.num_samples

    def state_dict(self) -> dict:
        return {"epoch": self._epoch, "seed": self.seed, "num_replicas": self.num_replicas, "rank": self.rank}

    def load_state_dict(self, state: dict) -> None:
        self._epoch = state.get("epoch", 0)
        self.seed = state.get("seed", self.seed)


class MixtureSampler(Sampler[int]):
    def __init__(self, cumulative_sizes: list[int], weights: list[float], num_replicas: int | None = None,
                 rank: int | None = None, shuffle: bool = True, seed: int = 0, drop_last: bool = True,
                 temperature: float = 1.0) -> None:
        self.num_replicas, self.rank = _replica_info(num_replicas, rank)
        n = len(cumulative_sizes) - 1
        self._sizes = [cumulative_sizes[i + 1] - cumulative_sizes[i] for i in range(n)]
        self._offsets = list(cumulative_sizes[:n])
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self._epoch = 0
        self._skip = 0
        self._set_quotas(weights, temperature, "MixtureSampler(weights=...)")

    def _set_quotas(self, weights: list[float], temperature: float, context: str) -> None:
        _validate_weights(weights, context)
        if len(weights) != len(self._sizes):
            raise ValueError(f"{context}: Expected {len(self._sizes)} weights, got {len(weights)}")
        if temperature != 1.0:
            logs = [math.log(max(w, 1e-12)) / temperature for w in weights]
            top = max(logs)
            scaled = [math.exp(v - top) for v in logs]
        else:
            scaled = list(weights)
        total = sum(scaled)
        self._probs = [s / total for s in scaled]
        per_rank = [(s // self.num_replicas) if self.drop_last else math.ceil(s / self.num_replicas)
                    for s in self._sizes]
        budget = sum(per_rank)
        quotas = [round(p * budget) for p in self._probs]
        gap = budget - sum(quotas)
        by_weight = sorted(range(len(quotas)), key=lambda i: -self._probs[i])
        for j in range(abs(gap)):
            quotas[by_weight[j % len(quotas)]] += 1 if gap > 0 else -1
        self._quotas = quotas
        self.num_samples = sum(quotas)

    def set_epoch(self, epoch: int) -> None:
        self._epoch = epoch

    def set_skip(self, skip: int) -> None:
        self._skip = max(0, skip)

    def __len__(self) -> int:
        return self.num_samples

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed + self._epoch)
        picked: list[int] = []
        for size, offset, quota in zip(self._sizes, self._offsets, self._quotas):
            if quota <= 0 or size == 0:
                continue
            order = torch.randperm(size, generator=g).tolist() if self.shuffle else list(range(size))
            if self.drop_last:
                order = order[: size - size % self.num_replicas]
            else:
                pad = (-len(order)) % self.num_replicas
                order += order[:pad]
            mine = order[self.rank :: self.num_replicas]
            if not mine:
                continue
            reps = -(-quota // len(mine))
            picked.extend(offset + i for i in (mine * reps)[:quota])
        if self.shuffle:
            perm = torch.randperm(len(picked), generator=g).tolist()
            picked = [picked[i] for i in perm]
        if self._skip:
            picked = picked[self._skip :]
            self._skip = 0
        return iter(picked)

    def update_weights(self, weights: list[float], temperature: float = 1.0) -> None:
        """Switch to new mixture weights (a training-phase transition); takes effect on the next ``iter``."""
        self._set_quotas(list(weights), temperature, "MixtureSampler.update_weights")

    def state_dict(self) -> dict:
        return {"epoch": self._epoch, "seed": self.seed, "num_replicas": self.num_replicas, "rank": self.rank,
                "probs": list(self._probs)}

    def load_state_dict(self, state: dict) -> None:
        self._epoch = state.get("epoch", 0)
        self.seed = state.get("seed", self.seed)
