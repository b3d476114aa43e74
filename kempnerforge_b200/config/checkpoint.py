"""Import path kept for code written against the reference layout (kempnerforge/config/checkpoint.py):
the classes live in ``config/sections.py``."""

from kempnerforge_b200.config.sections import CheckpointConfig, AsyncCheckpointMode, DynamicCheckpointWindow  # noqa: F401

__all__ = ['CheckpointConfig', 'AsyncCheckpointMode', 'DynamicCheckpointWindow']
