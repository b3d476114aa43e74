"""Graceful shutdown on SIGTERM / SIGUSR1.

The handler only sets a flag; the training loop polls it after every step, writes an emergency
checkpoint and leaves.  A daemon timer force-exits the process ``timeout_sec`` after the signal in
case a collective never returns (a cluster scheduler's kill would otherwise lose the checkpoint
window anyway).

Parity: kempnerforge/resilience/signal_handler.py:21-126.
"""

from __future__ import annotations

import logging
import os
import signal
import threading

log = logging.getLogger(__name__)
_SIGNALS = (signal.SIGTERM, signal.SIGUSR1)


class ShutdownHandler:
    def __init__(self, timeout_sec: float = 600.0) -> None:
        self.timeout_sec = timeout_sec
        self._requested = threading.Event()
        self._signal: int | None = None
        self._timer: threading.Timer | None = None
        self._previous: dict[int, object] = {}
        self._registered = False

    def register(self) -> None:
        if self._registered or threading.current_thread() is not threading.main_thread():
            return
        for sig in _SIGNALS:
            self._previous[sig] = signal.signal(sig, self._on_signal)
        self._registered = True

    def unregister(self) -> None:
        if not self._registered:
            return
        for sig, prev in self._previous.items():
            signal.signal(sig, prev)
        self._previous.clear()
        self._registered = False
        self.finish()

    def _on_signal(self, signum, frame) -> None:
        if self._requested.is_set():
            return
        self._signal = signum
        self._requested.set()
        log.warning("received signal %d; will stop after the current step", signum)
        if self.timeout_sec > 0:
            self._timer = threading.Timer(self.timeout_sec, self._force_exit)
            self._timer.daemon = True
            self._timer.start()

    def _force_exit(self) -> None:
        log.error("graceful shutdown did not finish within %.0fs; exiting", self.timeout_sec)
        os._exit(1)

    def should_shutdown(self) -> bool:
        return self._requested.is_set()

    @property
    def shutdown_requested(self) -> bool:
        return self._requested.is_set()

    def request(self) -> None:
        """Programmatic equivalent of receiving a signal (used by tests and hooks)."""
        self._on_signal(signal.SIGUSR1, None)

    @property
    def signal_received(self) -> int | None:
        return self._signal

    def finish(self) -> None:
        """Cancel the force-exit timer once shutdown work is done."""
        if self._timer is not None:
            self._timer.cancel()
            self._timer = None
