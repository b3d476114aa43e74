"""Import path kept for code written against the reference layout (kempnerforge/config/distributed.py):
the classes live in ``config/sections.py``."""

from kempnerforge_b200.config.sections import DistributedConfig  # noqa: F401

__all__ = ['DistributedConfig']
