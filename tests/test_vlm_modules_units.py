"""Cross-attention, mixture-of-transformers attention, vision encoders and freeze helpers against plain fp32
formulations.  Mirrors tests/unit/test_cross_attention.py, test_mot.py, test_vision.py and test_freeze.py of
the reference."""

from __future__ import annotations

import math

import pytest
import torch
from torch import nn

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.sections import ModelConfig
from kempnerforge_b200.config.vlm import FreezeSpec, FreezeStage, VisionEncoderConfig, VLMConfig
from kempnerforge_b200.models.cross_attention import CrossAttention, CrossAttentionBlock
from kempnerforge_b200.models.mot import MoTAttention, MoTBlock, mot_warm_start_from_text_stack, text_key_to_mot_keys
from kempnerforge_b200.models.position import apply_rope, precompute_rope_frequencies
from kempnerforge_b200.models.vision import RandomVisionEncoder, VisionEncoder, build_vision_encoder
from kempnerforge_b200.training.freeze import apply_freeze_specs, canonical_freeze_meta, effective_freeze, freeze_params


def _cfg(**kw):
    base = dict(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48, max_seq_len=32)
    base.update(kw)
    return ModelConfig(**base)


def _sdpa(q, k, v, mask=None, causal=False):
    """(b, s, h, d) attention in fp32 with grouped KV heads expanded."""
    rep = q.shape[2] // k.shape[2]
    k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(q.shape[-1])
    if causal:
        t = torch.ones(q.shape[1], k.shape[1], dtype=torch.bool).tril()
        s = s.masked_fill(~t, float("-inf"))
    if mask is not None:
        s = s.masked_fill(~mask[:, None, None, :].bool(), float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", s.softmax(-1), v)


# --------------------------------------------------------------------------- cross attention
@pytest.mark.parametrize("heads,kv", [(4, 4), (4, 2), (4, 1)])
def test_cross_attention_matches_plain_formulation(heads, kv):
    torch.manual_seed(0)
    ca = CrossAttention(32, heads, kv)
    nn.init.normal_(ca.o_proj.weight, std=0.2)
    x, img = torch.randn(2, 5, 32), torch.randn(2, 7, 32)
    mask = torch.ones(2, 7, dtype=torch.bool)
    mask[1, 4:] = False
    hd = 32 // heads
    q = (x @ ca.q_proj.weight.t()).view(2, 5, heads, hd)
    k = (img @ ca.k_proj.weight.t()).view(2, 7, kv, hd)
    v = (img @ ca.v_proj.weight.t()).view(2, 7, kv, hd)
    for m in (None, mask):
        want = _sdpa(q, k, v, m).reshape(2, 5, -1) @ ca.o_proj.weight.t()
        got = ca(x, img, m)
        assert got.shape == (2, 5, 32) and got.dtype == x.dtype
        assert torch.allclose(got, want, atol=1e-5)


def test_cross_attention_mask_semantics():
    torch.manual_seed(1)
    ca = CrossAttention(32, 4, 2)
    nn.init.normal_(ca.o_proj.weight, std=0.2)
    x, img = torch.randn(1, 4, 32), torch.randn(1, 6, 32)
    full = ca(x, img)
    assert torch.allclose(ca(x, img, torch.ones(1, 6, dtype=torch.bool)), full, atol=1e-6)
    mask = torch.tensor([[1, 1, 0, 1, 1, 1]], dtype=torch.bool)
    assert torch.allclose(ca(x, img, mask), ca(x, img[:, mask[0]]), atol=1e-6)   # masking a key == removing it
    perm = torch.tensor([5, 3, 4, 0, 2, 1])
    assert torch.allclose(ca(x, img[:, perm]), full, atol=1e-6)                   # no causal order over image tokens
    assert not torch.allclose(ca(x, img + 1.0), full)


def test_cross_attention_gradients_match_plain_formulation():
    torch.manual_seed(2)
    ca = CrossAttention(32, 4, 2)
    nn.init.normal_(ca.o_proj.weight, std=0.2)
    x = torch.randn(1, 3, 32, requires_grad=True)
    img = torch.randn(1, 4, 32, requires_grad=True)
    ca(x, img).square().sum().backward()
    got = [x.grad.clone(), img.grad.clone()] + [p.grad.clone() for p in ca.parameters()]
    assert all(g.abs().sum() > 0 for g in got)
    x.grad = img.grad = None
    ca.zero_grad()
    q = (x @ ca.q_proj.weight.t()).view(1, 3, 4, 8)
    k = (img @ ca.k_proj.weight.t()).view(1, 4, 2, 8)
    v = (img @ ca.v_proj.weight.t()).view(1, 4, 2, 8)
    (_sdpa(q, k, v).reshape(1, 3, -1) @ ca.o_proj.weight.t()).square().sum().backward()
    want = [x.grad, img.grad] + [p.grad for p in ca.parameters()]
    for g, w in zip(got, want):
        assert torch.allclose(g, w, atol=1e-4, rtol=1e-4)


def test_cross_attention_block_starts_as_identity_and_learns():
    torch.manual_seed(3)
    blk = CrossAttentionBlock(_cfg())
    x, img = torch.randn(2, 5, 32), torch.randn(2, 3, 32)
    assert torch.equal(blk(x, img), x)          # zero-initialised output projections
    opt = torch.optim.SGD(blk.parameters(), lr=0.5)
    blk(x, img).square().sum().backward()
    opt.step()
    assert not torch.equal(blk(x, img), x)
    frozen = CrossAttentionBlock(_cfg())
    for p in frozen.parameters():
        p.requires_grad_(False)
    assert not frozen(x, img).requires_grad


# --------------------------------------------------------------------------- mixture of transformers
def _rope(lengths, hd):
    cos, sin = precompute_rope_frequencies(hd, sum(lengths.values()))
    out, off = {}, 0
    for m, t in lengths.items():
        out[m] = (cos[off:off + t], sin[off:off + t])
        off += t
    return out


def _mot(heads=4, kv=2, qk_norm=False):
    torch.manual_seed(4)
    att = MoTAttention(32, heads, kv, ("image", "text"), qk_norm=qk_norm)
    for m in att.modalities:
        nn.init.normal_(att.o_proj[m].weight, std=0.2)
    return att


def test_mot_attention_construction_rules():
    att = MoTAttention(32, 4, 2, ("image", "text"))
    assert all(torch.count_nonzero(att.o_proj[m].weight) == 0 for m in att.modalities)
    assert att.q_proj["image"].weight.data_ptr() != att.q_proj["text"].weight.data_ptr()
    assert att.q_norm is None and MoTAttention(32, 4, 2, ("image", "text"), qk_norm=True).q_norm is not None
    with pytest.raises(ValueError):
        MoTAttention(32, 4, 2, ())
    with pytest.raises(ValueError):
        MoTAttention(32, 4, 3, ("image", "text"))
    with pytest.raises(ValueError):
        att({"text": torch.zeros(1, 2, 32)}, _rope({"text": 2}, 8))


@pytest.mark.parametrize("heads,kv,qk_norm", [(4, 4, False), (4, 2, False), (4, 2, True)])
def test_mot_attention_matches_joint_attention_over_both_streams(heads, kv, qk_norm):
    att = _mot(heads, kv, qk_norm)
    streams = {"image": torch.randn(2, 3, 32), "text": torch.randn(2, 5, 32)}
    rope = _rope({"image": 3, "text": 5}, att.head_dim)
    got = att(streams, rope)
    hd = att.head_dim
    qs, ks, vs = [], [], []
    for m in att.modalities:
        x = streams[m]
        b, t, _ = x.shape
        q = (x @ att.q_proj[m].weight.t()).view(b, t, heads, hd)
        k = (x @ att.k_proj[m].weight.t()).view(b, t, kv, hd)
        v = (x @ att.v_proj[m].weight.t()).view(b, t, kv, hd)
        if qk_norm:
            q, k = att.q_norm[m](q), att.k_norm[m](k)
        cos, sin = rope[m]
        qs.append(apply_rope(q, cos, sin))
        ks.append(apply_rope(k, cos, sin))
        vs.append(v)
    out = _sdpa(torch.cat(qs, 1), torch.cat(ks, 1), torch.cat(vs, 1), causal=True)
    off = 0
    for m in att.modalities:
        t = streams[m].shape[1]
        want = out[:, off:off + t].reshape(2, t, -1) @ att.o_proj[m].weight.t()
        assert got[m].shape == streams[m].shape and got[m].dtype == streams[m].dtype
        assert torch.allclose(got[m], want, atol=1e-5)
        off += t


def test_mot_streams_interact_through_attention_only():
    att = _mot()
    rope = _rope({"image": 3, "text": 5}, att.head_dim)
    img, txt = torch.randn(1, 3, 32), torch.randn(1, 5, 32)
    base = att({"image": img, "text": txt}, rope)
    other = att({"image": torch.randn(1, 3, 32), "text": txt}, rope)
    assert not torch.allclose(base["text"], other["text"])      # text queries see image keys
    later = att({"image": img, "text": txt + 1.0}, rope)
    assert torch.allclose(base["image"], later["image"], atol=1e-6)  # image comes first: causal, unaffected by text


def test_mot_gradients_reach_every_modality():
    att = _mot()
    rope = _rope({"image": 3, "text": 5}, att.head_dim)
    out = att({"image": torch.randn(1, 3, 32), "text": torch.randn(1, 5, 32)}, rope)
    sum(o.square().sum() for o in out.values()).backward()
    for name, p in att.named_parameters():
        assert p.grad is not None and p.grad.abs().sum() > 0, name


def test_mot_block_identity_at_init_keys_and_training():
    torch.manual_seed(5)
    cfg = _cfg()
    blk = MoTBlock(cfg, ("image", "text"), 0)
    rope = _rope({"image": 3, "text": 5}, cfg.head_dim)
    streams = {"image": torch.randn(2, 3, 32), "text": torch.randn(2, 5, 32)}
    out = blk(streams, rope)
    assert all(torch.equal(out[m], streams[m]) for m in streams)
    with pytest.raises(ValueError):
        blk({"text": streams["text"]}, rope)
    opt = torch.optim.SGD(blk.parameters(), lr=0.5)
    sum(o.square().sum() for o in out.values()).backward()
    opt.step()
    assert not torch.equal(blk(streams, rope)["text"], streams["text"])
    assert MoTBlock(_cfg(qk_norm=True), ("image", "text"), 0).attn.q_norm is not None


def test_text_keys_map_to_one_key_per_modality():
    mods = ("image", "text")
    assert text_key_to_mot_keys("layers.3.attention.q_proj.weight", mods) == [
        "layers.3.attn.q_proj.image.weight", "layers.3.attn.q_proj.text.weight"]
    assert text_key_to_mot_keys("layers.0.mlp.down_proj.weight", mods) == [
        "layers.0.mlp.image.down_proj.weight", "layers.0.mlp.text.down_proj.weight"]
    assert text_key_to_mot_keys("layers.1.attention_norm.weight", mods) == [
        "layers.1.attn_norm.image.weight", "layers.1.attn_norm.text.weight"]
    assert text_key_to_mot_keys("token_embedding.embedding.weight", mods) == ["token_embedding.embedding.weight"]
    assert "mot_norms.image.weight" in text_key_to_mot_keys("norm.weight", mods)


def test_mot_warm_start_copies_into_every_modality_and_is_idempotent():
    torch.manual_seed(6)
    cfg = _cfg()

    class Host(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleDict({"0": MoTBlock(cfg, ("image", "text"), 0)})
            self._mot_modalities = ("image", "text")

    host = Host()
    src = {"transformer.layers.0.attention.q_proj.weight": torch.randn(32, 32),
           "layers.0.mlp.up_proj.weight": torch.randn(48, 32),
           "layers.7.attention.q_proj.weight": torch.randn(32, 32)}      # layer the target does not have: skipped
    n = mot_warm_start_from_text_stack(host, src)
    att = host.layers["0"].attn
    for m in ("image", "text"):
        assert torch.equal(att.q_proj[m].weight, src["transformer.layers.0.attention.q_proj.weight"])
        assert torch.equal(host.layers["0"].mlp[m].up_proj.weight, src["layers.0.mlp.up_proj.weight"])
    assert n == 4 and mot_warm_start_from_text_stack(host, src) == 4
    with pytest.raises(ValueError, match="shape mismatch"):              # a wrong shape is never skipped
        mot_warm_start_from_text_stack(host, {"layers.0.attention.k_proj.weight": torch.randn(5, 5)})
    assert mot_warm_start_from_text_stack(nn.Linear(2, 2), src) == 0     # nothing to do on a non-MoT module


# --------------------------------------------------------------------------- vision encoders
def test_random_vision_encoder_contract():
    enc = RandomVisionEncoder(num_tokens=9, feature_dim=24)
    assert isinstance(enc, VisionEncoder) and (enc.num_tokens, enc.feature_dim) == (9, 24)
    a, b = torch.rand(2, 3, 32, 32), torch.rand(2, 3, 32, 32)
    fa = enc(a)
    assert fa.shape == (2, 9, 24) and fa.device == a.device
    assert torch.equal(enc(a), fa) and not torch.allclose(enc(b), fa)
    assert enc.double()(a).dtype == torch.double


def test_vision_encoder_registry_and_builder():
    assert {"random", "siglip2", "clip"} <= set(registry.list("vision_encoder"))
    enc = build_vision_encoder(VisionEncoderConfig(type="random", num_tokens=4, feature_dim=8))
    assert isinstance(enc, RandomVisionEncoder) and enc(torch.rand(1, 3, 16, 16)).shape == (1, 4, 8)
    assert build_vision_encoder(VisionEncoderConfig(type="random")).num_tokens == 16
    with pytest.raises((KeyError, ValueError)):
        registry.get("vision_encoder", "resnet")
    with pytest.raises(Exception):
        build_vision_encoder(VisionEncoderConfig(type="siglip2", path=""))   # nothing to load from an empty path


# --------------------------------------------------------------------------- freeze helpers
class _Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.vision_encoder = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4))
        self.adapter = nn.Linear(4, 4)
        self.transformer = nn.ModuleDict({"layers": nn.ModuleList([nn.Linear(4, 4)]), "head": nn.Linear(4, 4)})


_PATTERNS = {"vision_encoder": ["vision_encoder.*"], "adapter": ["adapter.*", "adapter"], "transformer": ["transformer.*"]}


def _frozen(model):
    return sorted(n for n, p in model.named_parameters() if not p.requires_grad)


def test_freeze_params_patterns_union_idempotent_and_unfreeze():
    m = _Toy()
    assert freeze_params(m, []) == 0 and _frozen(m) == []
    n = freeze_params(m, ["vision_encoder.*"])
    assert n == 2 * (16 + 4) and all(k.startswith("vision_encoder") for k in _frozen(m))   # elements flipped
    assert freeze_params(m, ["vision_encoder.*"]) == 0 and len(_frozen(m)) == 4            # nothing left to flip
    freeze_params(m, ["adapter.*", "transformer.head.*"])
    assert len(_frozen(m)) == 4 + 2 + 2
    freeze_params(m, ["vision_encoder.*"], frozen=False)
    assert not any(k.startswith("vision_encoder") for k in _frozen(m))
    freeze_params(m, ["*.bias"])
    assert all(not p.requires_grad for n_, p in m.named_parameters() if n_.endswith("bias"))


def test_apply_freeze_specs_aliases_and_errors():
    m = _Toy()
    counts = apply_freeze_specs(m, [FreezeSpec("vision_encoder", True), FreezeSpec("adapter", True),
                                    FreezeSpec("adapter", False)], _PATTERNS)
    assert counts["vision_encoder"] == 40 and not any(k.startswith("adapter") for k in _frozen(m))
    assert apply_freeze_specs(m, [FreezeSpec("vison_encoder", True)], _PATTERNS) == {"vison_encoder": 0}
    assert apply_freeze_specs(m, [FreezeSpec("adapter.weight", True)], _PATTERNS) == {"adapter.weight": 16}   # raw pattern


def test_canonical_freeze_meta_is_order_free_and_deduplicated():
    a = canonical_freeze_meta([FreezeSpec("b", True), FreezeSpec("a", False)])
    b = canonical_freeze_meta([FreezeSpec("a", False), FreezeSpec("b", True)])
    assert a == b == [{"module": "a", "frozen": False}, {"module": "b", "frozen": True}]
    both = canonical_freeze_meta([FreezeSpec("a", True), FreezeSpec("a", False), FreezeSpec("a", True)])
    assert both == [{"module": "a", "frozen": False}, {"module": "a", "frozen": True}]   # the set of pairs, sorted
    assert canonical_freeze_meta([]) == []


def test_effective_freeze_overlays_reached_stages():
    cfg = VLMConfig(freeze=[FreezeSpec("vision_encoder", True), FreezeSpec("adapter", True)],
                    freeze_schedule=[FreezeStage(10, (FreezeSpec("adapter", False),)),
                                     FreezeStage(20, (FreezeSpec("vision_encoder", False), FreezeSpec("adapter", True)))])
    state = lambda step: {s.module: s.frozen for s in effective_freeze(cfg, step)}  # noqa: E731
    assert state(0) == {"vision_encoder": True, "adapter": True}
    assert state(10) == {"vision_encoder": True, "adapter": False}
    assert state(25) == {"vision_encoder": False, "adapter": True}
    assert effective_freeze(None, 5) == []
    assert [s.module for s in effective_freeze(VLMConfig(), 0)] == ["vision_encoder"]
