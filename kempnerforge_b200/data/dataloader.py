"""A data loader whose position can be checkpointed.

State = epoch, batches already yielded in this epoch, sampler state.  On ``iter()`` the sampler is
told the epoch and how many samples to skip, so a resumed run sees exactly the batches the
interrupted run would have seen next; when an epoch ends the counters roll over and the next
``iter()`` starts the following epoch.

Parity: kempnerforge/data/dataloader.py:23-124.
"""

from __future__ import annotations

import torch
from torch.utils.data import DataLoader, Dataset, Sampler


class StatefulDataLoader:
    def __init__(self, dataset: Dataset, batch_size: int, sampler: Sampler | None = None, num_workers: int = 0,
                 pin_memory: bool = False, prefetch_factor: int | None = 2, drop_last: bool = True,
                 collate_fn=None, config=None) -> None:
        """Worker settings are given one by one, or as ``config=DataConfig`` (the reference's calling convention,
        kempnerforge/data/dataloader.py:53-64); a ``DataConfig`` passed as the fourth positional argument works too."""
        if config is None and not isinstance(num_workers, int):
            config, num_workers = num_workers, 0
        if config is not None:
            num_workers, pin_memory = int(config.num_workers), bool(config.pin_memory)
            prefetch_factor = config.prefetch_factor
        if sampler is None and not isinstance(dataset, torch.utils.data.IterableDataset):
            from kempnerforge_b200.data.sampler import DistributedSampler

            sampler = DistributedSampler(dataset)        # rank / world from the environment, seeded shuffle
        self.dataset, self.batch_size, self.sampler = dataset, batch_size, sampler
        kwargs = dict(batch_size=batch_size, sampler=sampler, num_workers=num_workers,
                      pin_memory=pin_memory and torch.cuda.is_available(), drop_last=drop_last,
                      collate_fn=collate_fn)
        if num_workers > 0:
            kwargs.update(prefetch_factor=prefetch_factor, persistent_workers=True)
        if isinstance(dataset, torch.utils.data.IterableDataset):
            kwargs.pop("sampler")
        self._loader = DataLoader(dataset, **kwargs)
        self._epoch = 0
        self._batches_yielded = 0
        self._iter = None

    def __iter__(self):
        if self.sampler is not None:
            if hasattr(self.sampler, "set_epoch"):
                self.sampler.set_epoch(self._epoch)
            if hasattr(self.sampler, "set_skip"):
                self.sampler.set_skip(self._batches_yielded * self.batch_size)
        self._iter = iter(self._loader)
        return self

    def __next__(self):
        if self._iter is None:
            iter(self)
        try:
            batch = next(self._iter)
        except StopIteration:
            self._epoch += 1
            self._batches_yielded = 0
            self._iter = None
            raise
        self._batches_yielded += 1
        return batch

    def __len__(self) -> int:
        return len(self._loader)

    def state_dict(self) -> dict:
        state = {"epoch": self._epoch, "batches_yielded": self._batches_yielded}
        if self.sampler is not None and hasattr(self.sampler, "state_dict"):
            state["sampler"] = self.sampler.state_dict()
        if hasattr(self.dataset, "state_dict"):
            state["dataset"] = self.dataset.state_dict()
        return state

    def load_state_dict(self, state: dict) -> None:
        self._epoch = state.get("epoch", 0)
        self._batches_yielded = state.get("batches_yielded", 0)
        if self.sampler is not None and "sampler" in state and hasattr(self.sampler, "load_state_dict"):
            self.sampler.load_state_dict(state["sampler"])
        if "dataset" in state and hasattr(self.dataset, "load_state_dict"):
            self.dataset.load_state_dict(state["dataset"])
        self._iter = None
