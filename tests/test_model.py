"""Model numerics on CPU: ops against closed forms, module wiring, state-dict keys, MoE, generation."""

import math

import pytest
import torch

from kempnerforge_b200.config import ModelConfig
from kempnerforge_b200.models import (
    Attention,
    KVCache,
    MoEMLP,
    RMSNorm,
    SigmoidTopKRouter,
    SoftmaxTopKRouter,
    SwiGLUMLP,
    Transformer,
    apply_capacity,
    apply_rope,
    build_mlp,
    build_moe,
    precompute_rope_frequencies,
)
from kempnerforge_b200.ops import ref

TINY = dict(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=256, max_seq_len=64)


def test_rmsnorm_matches_formula():
    x = torch.randn(3, 5, 32)
    n = RMSNorm(32, eps=1e-5)
    with torch.no_grad():
        n.weight.copy_(torch.rand(32) + 0.5)
    want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * n.weight
    assert torch.allclose(n(x), want, atol=1e-6)


def test_rope_properties():
    cos, sin = precompute_rope_frequencies(16, 32, 10000.0)
    assert cos.shape == (32, 8) and cos.dtype == torch.float32
    x = torch.randn(2, 32, 3, 16)
    y = apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)  # a rotation preserves length
    assert torch.allclose(y[:, 0], x[:, 0], atol=1e-6)  # position 0 is the identity
    # relative property: <rope(q, m), rope(k, n)> depends on m - n only
    q, k = torch.randn(1, 1, 1, 16), torch.randn(1, 1, 1, 16)
    def dot(m, n):
        qm = apply_rope(q.expand(1, 32, 1, 16), cos, sin)[0, m, 0]
        kn = apply_rope(k.expand(1, 32, 1, 16), cos, sin)[0, n, 0]
        return (qm * kn).sum()
    assert torch.allclose(dot(5, 3), dot(12, 10), atol=1e-5)


def test_attention_reference_matches_sdpa_and_gqa():
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 16, 4, 8), torch.randn(2, 16, 2, 8), torch.randn(2, 16, 2, 8)
    got = ref.attention(q, k, v, causal=True)
    kk, vv = k.repeat_interleave(2, dim=2), v.repeat_interleave(2, dim=2)
    want = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True).transpose(1, 2)
    assert torch.allclose(got, want, atol=1e-5)


def test_attention_doc_mask_isolates_documents():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 8, 2, 4), torch.randn(1, 8, 2, 4), torch.randn(1, 8, 2, 4)
    doc = torch.tensor([[0, 0, 0, 1, 1, 1, 1, 2]])
    out = ref.attention(q, k, v, causal=True, doc_ids=doc)
    # the second document alone gives the same result for its tokens
    alone = ref.attention(q[:, 3:7], k[:, 3:7], v[:, 3:7], causal=True)
    assert torch.allclose(out[:, 3:7], alone, atol=1e-6)


def test_attention_module_kv_cache_matches_full():
    torch.manual_seed(0)
    att = Attention(32, 4, 2)
    cos, sin = precompute_rope_frequencies(8, 16)
    x = torch.randn(1, 6, 32)
    full = att(x, cos[:6], sin[:6])
    cache = KVCache(1, 16, 2, 8, torch.float32, "cpu")
    first = att(x[:, :4], cos[:4], sin[:4], kv_cache=cache)
    assert torch.allclose(first, full[:, :4], atol=1e-5)
    for t in (4, 5):
        step = att(x[:, t : t + 1], cos[t : t + 1], sin[t : t + 1], kv_cache=cache)
        assert torch.allclose(step, full[:, t : t + 1], atol=1e-5)
    assert cache.seq_len == 6


def test_attention_capture_weights_and_qk_norm():
    att = Attention(32, 4, 4, qk_norm=True)
    att.capture_attention_weights = True
    cos, sin = precompute_rope_frequencies(8, 8)
    att(torch.randn(2, 8, 32), cos, sin)
    w = att.last_attention_weights
    assert w.shape == (2, 4, 8, 8)
    assert torch.allclose(w.sum(-1), torch.ones(2, 4, 8), atol=1e-5)
    assert torch.all(torch.triu(w, 1) == 0)


def test_swiglu_mlp_formula():
    m = SwiGLUMLP(16, 40)
    x = torch.randn(3, 16)
    want = (torch.nn.functional.silu(x @ m.gate_proj.weight.T) * (x @ m.up_proj.weight.T)) @ m.down_proj.weight.T
    assert torch.allclose(m(x), want, atol=1e-6)
    assert type(build_mlp(16, 32, "gelu")).__name__ == "StandardMLP"
    with pytest.raises(ValueError):
        build_mlp(16, 32, "tanh")


def test_transformer_state_dict_keys_and_param_count():
    cfg = ModelConfig(**TINY)
    m = Transformer(cfg)
    keys = set(m.state_dict())
    for k in ("token_embedding.embedding.weight", "layers.0.attention_norm.weight", "layers.1.attention.q_proj.weight",
              "layers.0.mlp.gate_proj.weight", "layers.0.mlp_norm.weight", "norm.weight", "output_head.proj.weight"):
        assert k in keys
    assert sum(p.numel() for p in m.parameters()) == cfg.num_params_estimate
    tied = Transformer(ModelConfig(**TINY, tie_embeddings=True))
    assert tied.output_head.proj.weight is tied.token_embedding.embedding.weight


def test_init_scaling_of_residual_projections():
    torch.manual_seed(0)
    cfg = ModelConfig(dim=256, n_layers=8, n_heads=4, vocab_size=512, max_seq_len=32)
    m = Transformer(cfg)
    std_q = m.layers["0"].attention.q_proj.weight.std().item()
    std_o = m.layers["0"].attention.o_proj.weight.std().item()
    assert abs(std_q - 0.02) < 2e-3
    assert abs(std_o - 0.02 / math.sqrt(16)) < 1e-3
    assert torch.all(m.norm.weight == 1)


def test_forward_backward_and_fused_loss_equals_plain_ce():
    torch.manual_seed(0)
    m = Transformer(ModelConfig(**TINY))
    tok = torch.randint(0, 256, (2, 33))
    labels = tok[:, 1:].clone()
    labels[0, :5] = -100
    fused = m.compute_loss(tok[:, :-1], labels, z_loss_weight=1e-3, chunk_tokens=16)
    logits = m(tok[:, :-1])
    plain = ref.cross_entropy(logits, labels, z_loss_weight=1e-3)
    assert torch.allclose(fused, plain, atol=1e-5)
    fused.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())


def test_activation_checkpointing_same_gradients():
    torch.manual_seed(0)
    m = Transformer(ModelConfig(**TINY))
    tok = torch.randint(0, 256, (2, 17))
    m.compute_loss(tok[:, :-1], tok[:, 1:]).backward()
    base = {n: p.grad.clone() for n, p in m.named_parameters()}
    for mode in ("full", "selective"):
        m.zero_grad()
        for blk in m.layers.values():
            blk.ac_mode = mode
        m.train()
        m.compute_loss(tok[:, :-1], tok[:, 1:]).backward()
        for n, p in m.named_parameters():
            assert torch.allclose(p.grad, base[n], atol=1e-6), (mode, n)


def test_forward_argument_rules():
    from kempnerforge_b200.models import ModalityContext

    m = Transformer(ModelConfig(**TINY))
    with pytest.raises(ValueError):
        m()
    with pytest.raises(ValueError):
        ModalityContext(inputs_embeds=torch.zeros(1, 2, 64), prefix_embeds=torch.zeros(1, 2, 64))
    with pytest.raises(ValueError):
        ModalityContext(image_mask=torch.ones(1, 2))
    caches = [KVCache(1, 8, 2, 16, torch.float32, "cpu") for _ in range(2)]
    with pytest.raises(ValueError):
        m(torch.zeros(1, 2, dtype=torch.long), kv_caches=caches, modality=ModalityContext(output_slice=slice(0, 1)))
    out = m(torch.zeros(1, 4, dtype=torch.long), modality=ModalityContext(output_slice=slice(1, 3)))
    assert out.shape == (1, 2, 256)


# ------------------------------------------------------------------ routers / MoE
def test_softmax_router_semantics():
    torch.manual_seed(0)
    r = SoftmaxTopKRouter(16, 8, 2)
    x = torch.randn(64, 16)
    w, idx = r(x)
    assert w.shape == (64, 2) and idx.shape == (64, 2)
    assert torch.allclose(w.sum(-1), torch.ones(64), atol=1e-6)
    assert r.expert_counts.sum().item() == 128
    probs = torch.softmax(r.gate(x), -1)
    f = r.expert_counts / 128
    assert torch.allclose(r.aux_loss, 8 * (f * probs.mean(0)).sum(), atol=1e-6)
    assert torch.allclose(r.z_loss, torch.logsumexp(r.gate(x), -1).pow(2).mean(), atol=1e-6)


def test_sigmoid_router_bias_balancing():
    torch.manual_seed(0)
    r = SigmoidTopKRouter(16, 4, 1)
    with torch.no_grad():
        r.gate.weight.zero_()
        r.gate.weight[0] = 1.0  # expert 0 always wins for positive-sum inputs
    x = torch.rand(128, 16)
    r.train()
    b0 = r.expert_bias.clone()
    for _ in range(20):
        r(x)
    assert r.expert_bias[0] < b0[0] and r.expert_bias[1] > b0[1]
    r.eval()
    b = r.expert_bias.clone()
    r(x)
    assert torch.equal(b, r.expert_bias)  # no balancing outside training
    r.bias_schedule = "cosine_decay"
    r.set_step(100, 100)
    assert abs(r._effective_bias_rate()) < 1e-9
    r.bias_schedule = "linear_warmup"
    r.set_step(5, 100)
    assert abs(r._effective_bias_rate() - 0.5e-3) < 1e-9


def test_capacity_keeps_first_tokens_per_slot():
    idx = torch.tensor([[0], [0], [0], [1]])
    w = torch.ones(4, 1)
    w2, _ = apply_capacity(w, idx, num_experts=2, capacity_factor=1.0)  # cap = ceil(4*1/2) = 2
    assert w2.flatten().tolist() == [1, 1, 0, 1]


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("router", ["softmax_topk", "sigmoid_topk"])
def test_moe_matches_per_token_loop(packed, router):
    torch.manual_seed(0)
    moe = build_moe(16, 32, num_experts=4, top_k=2, router_type=router, shared_experts=1, packed_experts=packed)
    moe.eval()
    x = torch.randn(2, 5, 16)
    got = moe(x)
    xf = x.reshape(-1, 16)
    w, idx = moe.router(xf)
    want = torch.zeros_like(xf)
    for t in range(xf.shape[0]):
        for s in range(2):
            e = idx[t, s].item()
            if packed:
                h = torch.nn.functional.silu(xf[t] @ moe.gate_w[e]) * (xf[t] @ moe.up_w[e])
                y = h @ moe.down_w[e]
            else:
                y = moe.experts[e](xf[t : t + 1])[0]
            want[t] += w[t, s] * y
    want = want + moe.shared_expert(xf)
    assert torch.allclose(got.reshape(-1, 16), want, atol=1e-5)
    got.sum().backward()
    names = [n for n, p in moe.named_parameters() if p.grad is None]
    assert names == [] or names == ["router.expert_bias"] or all("expert_bias" in n for n in names)


def test_moe_transformer_accessors_and_keys():
    cfg = ModelConfig(**TINY, num_experts=4, moe_top_k=2, moe_frequency=2, moe_router="sigmoid_topk", moe_shared_experts=2)
    m = Transformer(cfg)
    assert isinstance(m.layers["1"].mlp, MoEMLP) and not isinstance(m.layers["0"].mlp, MoEMLP)
    keys = set(m.state_dict())
    assert "layers.1.mlp.router.gate.weight" in keys and "layers.1.mlp.router.expert_bias" in keys
    assert "layers.1.mlp.router.expert_ema" in keys and "layers.1.mlp.experts.3.down_proj.weight" in keys
    assert "layers.1.mlp.shared_expert.up_proj.weight" in keys
    m(torch.randint(0, 256, (2, 8)))
    assert set(m.get_expert_counts()) == {1}
    assert m.get_moe_router_z_loss().item() > 0
    m.set_moe_step(3, 10)
    assert m.layers["1"].mlp.router._step == 3
    # the estimate counts two shared experts (one MLP is built) and omits the 4-element router bias
    assert sum(p.numel() for p in m.parameters()) == cfg.num_params_estimate - 3 * 64 * cfg.computed_expert_ffn_hidden_dim + 4


def test_generate_greedy_matches_full_forward():
    from kempnerforge_b200.models.generate import generate

    torch.manual_seed(0)
    m = Transformer(ModelConfig(**TINY)).eval()
    prompt = torch.randint(0, 256, (1, 5))
    out = generate(m, prompt, max_new_tokens=4, temperature=0.0)
    assert out.shape == (1, 9)
    seq = prompt.clone()
    for _ in range(4):
        nxt = m(seq)[:, -1].argmax(-1, keepdim=True)
        seq = torch.cat([seq, nxt], dim=1)
    assert torch.equal(out, seq)


def test_moe_blocks_keep_the_op_by_op_attention_path_off_the_gpu():
    """The fused attention sub-layer node is a GPU path: on CPU tensors its guard says no and the block's output is the
    plain residual formulation; the router's gate projection equals its ``nn.Linear``."""
    from kempnerforge_b200.models.router import build_router
    from kempnerforge_b200.ops import fused_block

    torch.manual_seed(0)
    cfg = ModelConfig(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, max_seq_len=32, ffn_hidden_dim=128,
                      num_experts=4, moe_top_k=2)
    model = Transformer(cfg)
    blk = next(iter(model.layers.values()))
    x = torch.randn(2, 16, 64)
    assert not fused_block.attn_half_supported(blk, x, None, None, None)
    cos, sin = model._rope_cos[:16], model._rope_sin[:16]
    want = x + blk.attention(blk.attention_norm(x), cos, sin)
    want = want + blk.mlp(blk.mlp_norm(want))
    assert torch.allclose(blk(x, cos, sin), want, atol=1e-6)
    router = build_router("softmax_topk", 64, 8, 2)
    tokens = torch.randn(10, 64)
    weights, indices = router(tokens)
    probs = torch.softmax(router.gate(tokens).float(), dim=-1)
    top_w, top_i = torch.topk(probs, 2, dim=-1)
    assert torch.equal(indices, top_i) and torch.allclose(weights, top_w / top_w.sum(-1, keepdim=True), atol=1e-6)
