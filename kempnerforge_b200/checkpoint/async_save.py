"""Synchronous / asynchronous hand-off to ``torch.distributed.checkpoint``.

``async`` stages tensors to host memory and writes in a background thread; ``async_with_pinned_mem``
additionally keeps a pinned staging cache alive between saves so the device-to-host copy runs at
full PCIe speed and without re-allocating.  A new save first waits for the previous one.

Parity: kempnerforge/checkpoint/async_save.py:38-73 (the reference treats both asynchronous modes
alike; here the pinned mode really pins).
"""

from __future__ import annotations

import logging
from concurrent.futures import Future

import torch.distributed.checkpoint as dcp

log = logging.getLogger(__name__)


class AsyncCheckpointer:
    def __init__(self, mode: str = "disabled", process_group=None) -> None:
        self.mode = str(mode)
        self.process_group = process_group
        self._future: Future | None = None
        self._stager = None

    @property
    def is_async(self) -> bool:
        return self.mode in ("async", "async_with_pinned_mem")

    def _pinned_stager(self):
        if self._stager is None:
            try:
                from torch.distributed.checkpoint.staging import DefaultStager, StagingOptions

                self._stager = DefaultStager(StagingOptions(use_pinned_memory=True, use_shared_memory=False,
                                                            use_async_staging=False, use_non_blocking_copy=True))
            except Exception as exc:  # older layouts of the staging API
                log.warning("pinned staging unavailable (%s); using default staging", exc)
                self._stager = False
        return self._stager or None

    def save(self, state_dict: dict, checkpoint_id: str, process_group=None) -> None:
        self.wait()
        pg = process_group or self.process_group
        if not self.is_async:
            dcp.save(state_dict, checkpoint_id=checkpoint_id, process_group=pg)
            log.info("Sync checkpoint saved: %s", checkpoint_id)
            return
        kwargs = {}
        if self.mode == "async_with_pinned_mem":
            stager = self._pinned_stager()
            if stager is not None:
                kwargs["async_stager"] = stager
        try:
            result = dcp.async_save(state_dict, checkpoint_id=checkpoint_id, process_group=pg, **kwargs)
        except TypeError:
            result = dcp.async_save(state_dict, checkpoint_id=checkpoint_id, process_group=pg)
        self._future = getattr(result, "upload_completion", result)
        log.info("Async checkpoint started: %s", checkpoint_id)

    def wait(self) -> None:
        if self._future is not None:
            self._future.result()
            self._future = None

    @property
    def is_pending(self) -> bool:
        """True from ``save`` until ``wait`` has collected the result (whether or not the write has finished)."""
        return self._future is not None

    @property
    def pending(self) -> bool:
        return self._future is not None and not self._future.done()
