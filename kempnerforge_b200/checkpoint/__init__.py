"""Checkpointing: DCP tensor state, train state, asynchronous saves, retention, auto-resume."""

from kempnerforge_b200.checkpoint.async_save import AsyncCheckpointer
from kempnerforge_b200.checkpoint.manager import (
    CheckpointManager,
    UntrustedCheckpointError,
    check_trusted_file,
    load_optimizer_state_dict,
    model_state_dict,
    optimizer_state_dict,
)
from kempnerforge_b200.checkpoint.state import build_train_state, get_rng_state, restore_train_state, set_rng_state

__all__ = [n for n in dir() if not n.startswith("_")]
