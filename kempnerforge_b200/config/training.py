"""Import path kept for code written against the reference layout (kempnerforge/config/training.py):
the classes live in ``config/sections.py``."""

from kempnerforge_b200.config.sections import TrainConfig  # noqa: F401

__all__ = ['TrainConfig']
