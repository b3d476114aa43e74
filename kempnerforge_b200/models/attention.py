"""Grouped-query attention with rotary embeddings.

One GEMM produces q, k and v (their weights are adjacent in the block's flat
parameter buffer), one kernel rotates the q and k heads in place of the six
elementwise ops of a naive RoPE, and the attention kernel reads KV head
``h // (n_heads // n_kv_heads)`` directly, so grouped KV heads are never
expanded.  Document masks are evaluated inside the kernel from per-token ids;
no (S, S) mask tensor is built on the native path.

Parity: kempnerforge/model/attention.py:29-280 (parameter names q/k/v/o_proj,
optional per-head q_norm/k_norm applied before RoPE, KV cache for decoding,
``capture_attention_weights`` / ``last_attention_weights`` for inspection,
causal / document / key-padding masks, scale 1/sqrt(head_dim)).
"""

from __future__ import annotations

import torch
from torch import nn

from kempnerforge_b200.models.norm import RMSNorm
from kempnerforge_b200.ops import functional as F
from kempnerforge_b200.ops import ref


class KVCache:
    """Pre-allocated keys/values for incremental decoding, stored (batch, position, kv_head, head_dim)."""

    def __init__(self, batch_size, max_seq_len, n_kv_heads, head_dim, dtype, device) -> None:
        shape = (batch_size, max_seq_len, n_kv_heads, head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.seq_len = 0

    def update(self, k_new: torch.Tensor, v_new: torch.Tensor):
        """Append (batch, new, kv_head, head_dim) entries; returns views over everything cached so far."""
        end = self.seq_len + k_new.shape[1]
        if end > self.k.shape[1]:
            raise ValueError(f"KV cache overflow: {end} > {self.k.shape[1]}")
        self.k[:, self.seq_len : end] = k_new
        self.v[:, self.seq_len : end] = v_new
        self.seq_len = end
        return self.k[:, :end], self.v[:, :end]

    def reset(self) -> None:
        self.seq_len = 0


class Attention(nn.Module):
    def __init__(
        self,
        dim: int,
        n_heads: int,
        n_kv_heads: int,
        head_dim: int | None = None,
        qk_norm: bool = False,
        sdpa_backend: str = "auto",
    ) -> None:
        super().__init__()
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim or dim // n_heads
        self.n_rep = n_heads // n_kv_heads
        self.sdpa_backend = sdpa_backend
        hd = self.head_dim
        self.q_proj = nn.Linear(dim, n_heads * hd, bias=False)
        self.k_proj = nn.Linear(dim, n_kv_heads * hd, bias=False)
        self.v_proj = nn.Linear(dim, n_kv_heads * hd, bias=False)
        self.o_proj = nn.Linear(n_heads * hd, dim, bias=False)
        self.q_norm = RMSNorm(hd) if qk_norm else None
        self.k_norm = RMSNorm(hd) if qk_norm else None
        self.capture_attention_weights = False
        self.last_attention_weights: torch.Tensor | None = None
        self.tp = None  # TPContext when q/k/v are column-sharded and o row-sharded

    def forward(
        self,
        x: torch.Tensor,
        rope_cos: torch.Tensor,
        rope_sin: torch.Tensor,
        kv_cache: KVCache | None = None,
        doc_ids: torch.Tensor | None = None,
        key_padding_mask: torch.Tensor | None = None,
    ) -> torch.Tensor:
        qkv_w = [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight]
        qkv = None
        if self.tp is not None:
            qkv = self.tp.column_linear(x, qkv_w)  # gathers the sequence shards (inside the GEMM when it can)
            b, s = qkv.shape[0], qkv.shape[1]
        else:
            b, s, _ = x.shape
        # local head counts follow the weight shapes so a tensor-parallel shard works unchanged
        hd = self.head_dim
        h = self.q_proj.weight.shape[0] // hd
        hkv = self.k_proj.weight.shape[0] // hd
        if qkv is None:
            qkv = F.fused_linear(x, qkv_w)
        qkv = qkv.view(b, s, h + 2 * hkv, hd)
        if self.q_norm is not None:
            qkv = torch.cat(
                [self.q_norm(qkv[:, :, :h]), self.k_norm(qkv[:, :, h : h + hkv]), qkv[:, :, h + hkv :]], dim=2
            )
        qkv = F.rope(qkv, rope_cos, rope_sin, n_rot_heads=h + hkv)
        q, k, v = qkv[:, :, :h], qkv[:, :, h : h + hkv], qkv[:, :, h + hkv :]
        if kv_cache is not None:
            k, v = kv_cache.update(k, v)
        causal = kv_cache is None or s > 1
        if self.capture_attention_weights:
            out, probs = ref.attention(q, k, v, causal, doc_ids, key_padding_mask, return_weights=True)
            self.last_attention_weights = probs.detach()
        else:
            out = F.attention(q, k, v, causal=causal, doc_ids=doc_ids, key_padding_mask=key_padding_mask)
        if self.tp is not None:
            return self.tp.row_linear(out.reshape(b, s, h * hd), self.o_proj.weight)
        return F.linear(out.reshape(b, s, h * hd), self.o_proj.weight)
