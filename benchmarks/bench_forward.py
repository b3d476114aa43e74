"""Forward / forward+backward of the 125 M model, attention over sequence lengths, the SwiGLU MLP.
Parity: benchmarks/bench_forward.py:26-108 in the reference (same cases and shapes)."""

from __future__ import annotations

import torch

from benchmarks._common import batch_shape, bench_model_config, dtype_for
from benchmarks.runner import Case, print_results, run_suite

SUITE = "forward"


def cases(device: torch.device):
    from kempnerforge_b200.models.attention import Attention
    from kempnerforge_b200.models.mlp import build_mlp
    from kempnerforge_b200.models.position import precompute_rope_frequencies
    from kempnerforge_b200.models.transformer import Transformer

    cfg = bench_model_config(device)
    dt = dtype_for(device)
    b, s = batch_shape(device)
    model = Transformer(cfg).to(device=device, dtype=dt)
    ids = torch.randint(0, cfg.vocab_size, (b, s), device=device)
    labels = torch.randint(0, cfg.vocab_size, (b, s), device=device)

    def fwd():
        with torch.no_grad():
            model(ids)

    def fwd_bwd():
        loss = model.compute_loss(ids, labels)
        (loss[0] if isinstance(loss, tuple) else loss).backward()
        model.zero_grad(set_to_none=True)

    size = f"{sum(p.numel() for p in model.parameters()) / 1e6:.0f}M"
    yield Case(f"forward ({size}, bs={b}, seq={s})", fwd, tokens_per_iter=b * s)
    yield Case(f"forward+backward, fused head+loss ({size})", fwd_bwd, tokens_per_iter=b * s)

    hd = cfg.dim // cfg.n_heads
    attn = Attention(cfg.dim, cfg.n_heads, cfg.n_kv_heads).to(device=device, dtype=dt)
    cos, sin = precompute_rope_frequencies(hd, cfg.max_seq_len)
    cos, sin = cos.to(device), sin.to(device)
    for seq in ([512, 1024, 2048] if device.type == "cuda" else [64, 128]):
        x = torch.randn(b, seq, cfg.dim, device=device, dtype=dt)

        def attn_fn(x=x, seq=seq):
            with torch.no_grad():
                attn(x, cos[:seq], sin[:seq])

        # causal attention FLOPs: QK^T and PV, half of the square each
        yield Case(f"attention block (seq={seq})", attn_fn, tokens_per_iter=b * seq,
                   flops_per_iter=2 * 2 * b * cfg.n_heads * seq * seq * hd / 2 + 2 * b * seq * cfg.dim * cfg.dim * 4)

    mlp = build_mlp(cfg.dim, cfg.computed_ffn_hidden_dim, "silu").to(device=device, dtype=dt)
    xm = torch.randn(b, s, cfg.dim, device=device, dtype=dt)

    def mlp_fn():
        with torch.no_grad():
            mlp(xm)

    yield Case("MLP (SwiGLU)", mlp_fn, tokens_per_iter=b * s,
               flops_per_iter=2 * b * s * cfg.dim * cfg.computed_ffn_hidden_dim * 3)


if __name__ == "__main__":
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    print_results(run_suite(SUITE, dev), "forward")
