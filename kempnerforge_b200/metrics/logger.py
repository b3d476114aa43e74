"""Rank-aware logging.

Only rank 0 prints by default; every record carries ``[rank r]``; colours are dropped when
``NO_COLOR`` is set or the stream is not a terminal.  ``format_metrics`` renders the one-line
step summary ``[step N] k=v | k=v | ...`` that tools (and the end-to-end tests) parse.

Parity: kempnerforge/metrics/logger.py:29-156.
"""

from __future__ import annotations

import logging
import os
import sys

_COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m", "CRITICAL": "\033[35m"}
_RESET = "\033[0m"


def _rank() -> int:
    for key in ("RANK", "SLURM_PROCID"):
        if key in os.environ:
            try:
                return int(os.environ[key])
            except ValueError:
                pass
    return 0


class RankFilter(logging.Filter):
    """Let records through on rank 0 only (or on every rank when ``all_ranks``)."""

    def __init__(self, all_ranks: bool = False, rank: int = 0) -> None:
        super().__init__()
        self.all_ranks = all_ranks
        self.allowed_rank = rank

    def filter(self, record: logging.LogRecord) -> bool:
        return self.all_ranks or _rank() == self.allowed_rank or record.levelno >= logging.ERROR


def _supports_color() -> bool:
    """Colour only on an interactive stream and never when NO_COLOR is set."""
    if os.environ.get("NO_COLOR"):
        return False
    stream = sys.stdout
    return bool(getattr(stream, "isatty", None)) and stream.isatty()


class RankFormatter(logging.Formatter):
    def __init__(self, use_color: bool | None = None) -> None:
        super().__init__()
        self.use_color = _supports_color() if use_color is None else (bool(use_color) and _supports_color())

    def format(self, record: logging.LogRecord) -> str:
        level = record.levelname
        if self.use_color and level in _COLORS:
            level = f"{_COLORS[level]}{level}{_RESET}"
        stamp = self.formatTime(record, "%H:%M:%S")
        msg = record.getMessage()
        if record.exc_info:
            msg += "\n" + self.formatException(record.exc_info)
        return f"{stamp} [rank {_rank()}] {level} {record.name}: {msg}"


_RankFilter, _RankFormatter = RankFilter, RankFormatter   # underscore spellings used by code written against the reference

_configured = False


def setup_logging(level: int | str = logging.INFO, all_ranks: bool = False) -> None:
    global _configured
    root = logging.getLogger("kempnerforge_b200")
    root.setLevel(level)
    if not _configured:
        handler = logging.StreamHandler(sys.stdout)
        handler.setFormatter(RankFormatter())
        handler.addFilter(RankFilter(all_ranks))
        root.addHandler(handler)
        root.propagate = False
        _configured = True


def _configure_root(rank_zero_only: bool = True) -> None:
    """Configure the package logger once (later calls do nothing)."""
    if not _configured:
        setup_logging(all_ranks=not rank_zero_only)


def get_logger(name: str = "kempnerforge_b200", rank_zero_only: bool = True) -> logging.Logger:
    """``rank_zero_only=False`` on the call that first configures logging lets every rank print."""
    if not _configured:
        setup_logging(all_ranks=not rank_zero_only)
    if not name.startswith("kempnerforge_b200"):
        name = f"kempnerforge_b200.{name}"
    return logging.getLogger(name)


def format_metrics(step: int, metrics: dict) -> str:
    """``[step 12] loss=2.3456 | lr=3.00e-04 | grad_norm=0.812 | tok/s=12,345 | mfu=41.2% | mem=10.1/180GB | step_time=0.53s``"""
    parts = []
    for key, val in metrics.items():
        if isinstance(val, str):                 # already rendered by the caller
            parts.append(f"{key}={val}")
            continue
        if key == "loss" or key.endswith("/loss") or key.startswith("loss/"):
            parts.append(f"{key}={val:.4f}")
        elif key == "lr":
            parts.append(f"lr={val:.2e}")
        elif key == "grad_norm":
            parts.append(f"grad_norm={val:.3f}")
        elif key == "tok/s":
            parts.append(f"tok/s={val:,.0f}")
        elif key == "mfu":
            parts.append(f"mfu={val:.1f}%")
        elif key == "mem":
            parts.append(f"mem={val}")
        elif key == "step_time":
            parts.append(f"step_time={val:.2f}s")
        else:
            parts.append(f"{key}={format_number(val)}")
    return f"[step {step}] " + " | ".join(parts)


def format_number(val) -> str:
    """Compact rendering of a metric value, same rules as the reference's log lines (kempnerforge/metrics/logger.py:
    120-140): integers (and whole floats from 1000 up) as 12.3k / 4.5M / 1.2B, tiny or huge floats in scientific
    notation, other floats with four decimals, anything else through ``str``."""
    if isinstance(val, bool) or not isinstance(val, (int, float)):
        return str(val)
    if isinstance(val, int) or (val == int(val) and abs(val) >= 1000 if val == val and abs(val) != float("inf") else False):
        n = int(val)
        mag = abs(n)
        if mag >= 1_000_000_000:
            return f"{n / 1e9:.1f}B"
        if mag >= 1_000_000:
            return f"{n / 1e6:.1f}M"
        if mag >= 1_000:
            return f"{n / 1e3:.0f}k" if mag % 1000 == 0 else f"{n / 1e3:.1f}k"
        return str(n)
    if val != val or abs(val) == float("inf"):
        return str(val)
    if abs(val) < 0.01 or abs(val) >= 1e6:
        return f"{val:.2e}"
    return f"{val:.4f}"


_format_number = format_number   # underscore spelling used by code written against the reference
