"""kempnerforge_b200: a Blackwell (sm_100a) native LLM / MoE pre-training framework."""

from kempnerforge_b200 import _reference_paths

__version__ = "0.1.0"

_reference_paths.install()   # kempnerforge_b200.model / .distributed / .config.<section> resolve to the modules here
