"""Every config class under one import path (kempnerforge/config/schema.py in the reference)."""

from kempnerforge_b200.config.job import JobConfig  # noqa: F401
from kempnerforge_b200.config.sections import *  # noqa: F401,F403
from kempnerforge_b200.config.vlm import *  # noqa: F401,F403
