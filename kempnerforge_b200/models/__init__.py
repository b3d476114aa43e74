"""Model zoo: decoder-only transformer (dense / MoE) and the vision-language wrappers."""

from kempnerforge_b200.models.attention import Attention, KVCache
from kempnerforge_b200.models.embedding import OutputHead, TokenEmbedding
from kempnerforge_b200.models.init import init_weights
from kempnerforge_b200.models.mlp import StandardMLP, SwiGLUMLP, build_mlp
from kempnerforge_b200.models.modality import ModalityContext
from kempnerforge_b200.models.moe import MoEMLP, apply_capacity, build_moe
from kempnerforge_b200.models.norm import RMSNorm, build_norm
from kempnerforge_b200.models.position import apply_rope, precompute_rope_frequencies
from kempnerforge_b200.models.router import SigmoidTopKRouter, SoftmaxTopKRouter, build_router
from kempnerforge_b200.models.transformer import Transformer, TransformerBlock

__all__ = [n for n in dir() if not n.startswith("_")]
