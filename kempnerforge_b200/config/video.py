"""Import path kept for code written against the reference layout (kempnerforge/config/video.py):
the classes live in ``config/vlm.py``."""

from kempnerforge_b200.config.vlm import VideoConfig  # noqa: F401

__all__ = ['VideoConfig']
