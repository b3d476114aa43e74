"""kempnerforge_b200: a Blackwell (sm_100a) native LLM / MoE pre-training framework."""

__version__ = "0.1.0"
