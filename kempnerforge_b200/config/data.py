"""Import path kept for code written against the reference layout (kempnerforge/config/data.py):
the classes live in ``config/sections.py``."""

from kempnerforge_b200.config.sections import DataConfig, DatasetSource, TrainingPhase  # noqa: F401

__all__ = ['DataConfig', 'DatasetSource', 'TrainingPhase']
