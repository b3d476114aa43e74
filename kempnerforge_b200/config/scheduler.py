"""Import path kept for code written against the reference layout (kempnerforge/config/scheduler.py):
the classes live in ``config/sections.py``."""

from kempnerforge_b200.config.sections import SchedulerConfig, SchedulerType  # noqa: F401

__all__ = ['SchedulerConfig', 'SchedulerType']
