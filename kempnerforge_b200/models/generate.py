"""Sampling and autoregressive generation with per-layer KV caches.

``sample``: temperature -> top-k -> top-p (nucleus) -> multinomial; temperature 0 is greedy.
``generate``: one prefill pass over the prompt, then one token per step against the caches.

Parity: kempnerforge/model/generate.py:15-131.
"""

from __future__ import annotations

import torch

from kempnerforge_b200.models.attention import KVCache


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
           generator: torch.Generator | None = None) -> torch.Tensor:
    """logits (batch, vocab) -> token ids (batch,); greedy at temperature 0."""
    if temperature <= 0:
        return logits.argmax(dim=-1)
    logits = logits.float() / temperature
    if top_k and top_k > 0:
        k = min(top_k, logits.shape[-1])
        kth = torch.topk(logits, k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        sorted_logits, order = torch.sort(logits, descending=True, dim=-1)
        probs = torch.softmax(sorted_logits, dim=-1)
        cum = probs.cumsum(dim=-1)
        drop = cum - probs >= top_p  # a token is kept while the mass before it is still below the threshold
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, order, sorted_logits)
    probs = torch.softmax(logits, dim=-1)
    return torch.multinomial(probs, 1, generator=generator).squeeze(-1)


@torch.no_grad()
def generate(model, prompt_tokens: torch.Tensor, max_new_tokens: int, temperature: float = 1.0, top_k: int = 0,
             top_p: float = 1.0, eos_token_id: int | None = None, generator: torch.Generator | None = None) -> torch.Tensor:
    cfg = model.config
    b, plen = prompt_tokens.shape
    total = plen + max_new_tokens
    if total > cfg.max_seq_len:
        raise ValueError(f"prompt ({plen}) + max_new_tokens ({max_new_tokens}) = {total} exceeds model max_seq_len "
                         f"({cfg.max_seq_len})")
    if max_new_tokens <= 0:
        return prompt_tokens
    param = next(model.parameters())
    hd = cfg.head_dim
    caches = [KVCache(b, total, layer.attention.k_proj.weight.shape[0] // hd, hd, param.dtype, param.device)
              for layer in model.layers.values()]
    was_training = model.training
    model.eval()
    logits = model(prompt_tokens, kv_caches=caches)
    out = prompt_tokens
    done = torch.zeros(b, dtype=torch.bool, device=prompt_tokens.device)
    for _ in range(total - plen):
        nxt = sample(logits[:, -1], temperature, top_k, top_p, generator)[:, None]
        if eos_token_id is not None:
            nxt = torch.where(done[:, None], torch.full_like(nxt, eos_token_id), nxt)
            done |= nxt.squeeze(-1) == eos_token_id
        out = torch.cat([out, nxt], dim=1)
        if out.shape[1] >= total or (eos_token_id is not None and bool(done.all())):
            break
        logits = model(nxt, kv_caches=caches)
    if was_training:
        model.train()
    return out
