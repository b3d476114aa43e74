"""MoE layer and MoE model: expert counts, top-k, packed vs per-expert weights, both routers.
Parity: benchmarks/bench_moe.py:17-129 in the reference."""

from __future__ import annotations

import torch

from benchmarks._common import batch_shape, bench_model_config, dtype_for
from benchmarks.runner import Case, print_results, run_suite

SUITE = "moe"


def cases(device: torch.device):
    from kempnerforge_b200.models.moe import build_moe
    from kempnerforge_b200.models.transformer import Transformer

    dt = dtype_for(device)
    b, s = batch_shape(device)
    dim = 768 if device.type == "cuda" else 128
    hidden = 2048 if device.type == "cuda" else 256
    x = torch.randn(b, s, dim, device=device, dtype=dt)
    grid = [(8, 2, "softmax_topk", False), (8, 2, "softmax_topk", True), (16, 2, "softmax_topk", True),
            (64, 6, "sigmoid_topk", True)]
    if device.type != "cuda":
        grid = grid[:2]
    for n_exp, k, router, packed in grid:
        layer = build_moe(dim, hidden, n_exp, k, router_type=router, packed_experts=packed).to(device=device, dtype=dt)

        def layer_fwd_bwd(layer=layer):
            xin = x.detach().requires_grad_(True)
            layer(xin).float().sum().backward()
            layer.zero_grad(set_to_none=True)

        tag = f"E={n_exp} k={k} {router.split('_')[0]}{' packed' if packed else ''}"
        yield Case(f"MoE layer fwd+bwd ({tag})", layer_fwd_bwd, tokens_per_iter=b * s,
                   flops_per_iter=3 * 2 * b * s * k * dim * hidden * 3)

    cfg = bench_model_config(device, num_experts=8, moe_top_k=2, moe_frequency=2, moe_packed_experts=True,
                             n_layers=4 if device.type == "cuda" else 2)
    model = Transformer(cfg).to(device=device, dtype=dt)
    ids = torch.randint(0, cfg.vocab_size, (b, s), device=device)
    labels = torch.randint(0, cfg.vocab_size, (b, s), device=device)

    def model_step():
        loss = model.compute_loss(ids, labels)
        loss = loss[0] if isinstance(loss, tuple) else loss
        (loss + 0.01 * model.get_moe_aux_loss()).backward()
        model.zero_grad(set_to_none=True)

    yield Case("MoE model fwd+bwd (8 experts, top-2, every 2nd layer)", model_step, tokens_per_iter=b * s)


if __name__ == "__main__":
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    print_results(run_suite(SUITE, dev), "moe")
