"""Numerics of every native kernel against a plain PyTorch fp32 formulation of the same op."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(got, want, rtol=2e-2, atol=2e-2):
    got, want = got.float(), want.float()
    err = (got - want).abs().max().item()
    ref = want.abs().max().item()
    assert torch.allclose(got, want, rtol=rtol, atol=atol * max(1.0, ref)), f"max err {err} (ref max {ref})"


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 264, 136), (1000, 776, 520), (2048, 1024, 4096)])
def test_gemm_all_layouts(native_lib, a_k, b_k, shape, mode):
    m, n, k = shape
    a = _rand(m, k, scale=0.5)
    b = _rand(n, k, scale=0.5)
    want = a.float() @ b.float().t()
    a_in = a if a_k else a.t().contiguous()
    b_in = b if b_k else b.t().contiguous()
    got = native_lib.gemm(a_in, b_in, a_kmajor=a_k, b_kmajor=b_k, mode=mode)
    torch.cuda.synchronize()
    assert native_lib.read_status() == 0
    _close(got, want, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_residual_epilogue(native_lib, mode):
    m, n, k = 520, 776, 264
    a, b = _rand(m, k, scale=0.5), _rand(n, k, scale=0.5)
    r = _rand(m, n)
    got = native_lib.gemm(a, b, residual=r, mode=mode)
    _close(got, a.float() @ b.float().t() + r.float())
    acc = _rand(m, n)
    want = acc.float() + a.float() @ b.float().t() + r.float()
    native_lib.gemm(a, b, out=acc, accumulate=True, residual=r, mode=mode)
    _close(acc, want)
    assert native_lib.read_status() == 0


@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_many_tiles_persistent(native_lib, mode):
    """More tiles than CTAs (several per persistent CTA, both accumulator buffers, ring wrap-around)."""
    m, n, k = 4096, 5120, 192
    a, b = _rand(m, k, scale=0.5), _rand(n, k, scale=0.5)
    got = native_lib.gemm(a, b, mode=mode)
    _close(got, a.float() @ b.float().t())
    assert native_lib.read_status() == 0


def test_gemm_accumulate_and_fp32_out(native_lib):
    m, n, k = 256, 512, 320
    a, b = _rand(m, k, scale=0.5), _rand(n, k, scale=0.5)
    base = torch.randn(m, n, device=DEV)
    out = base.clone()
    native_lib.gemm(a, b, out=out, accumulate=True)
    _close(out, base + a.float() @ b.float().t(), rtol=1e-2, atol=5e-3)
    out_bf = base.to(torch.bfloat16)
    want = out_bf.float() + a.float() @ b.float().t()
    native_lib.gemm(a, b, out=out_bf, accumulate=True)
    _close(out_bf, want)


def test_gemm_strided_rows(native_lib):
    big = _rand(512, 1024, scale=0.5)
    a = big[:, 256:768]  # row pitch 1024, 512 columns
    b = _rand(384, 512, scale=0.5)
    got = native_lib.gemm(a, b)
    _close(got, a.float() @ b.float().t())


@pytest.mark.parametrize("rows,d", [(7, 256), (300, 4096), (64, 5120), (33, 16384)])
def test_rmsnorm(native_lib, rows, d):
    from kempnerforge_b200.ops import ref

    x, w = _rand(rows, d), (1 + 0.1 * torch.randn(d, device=DEV)).to(torch.bfloat16)
    y, rstd = native_lib.rmsnorm_fwd(x, w, 1e-5)
    _close(y, ref.rmsnorm(x.float(), w.float(), 1e-5))
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    dy = _rand(rows, d)
    ref.rmsnorm(xf, wf, 1e-5).backward(dy.float())
    dx, dw = native_lib.rmsnorm_bwd(dy, x, w, rstd)
    _close(dx, xf.grad)
    _close(dw, wf.grad, rtol=3e-2, atol=3e-2)


def test_rope_roundtrip_and_reference(native_lib):
    from kempnerforge_b200.ops import ref

    b, s, h, hd = 2, 96, 6, 128
    x = _rand(b, s, h, hd)
    cos, sin = ref.rope_tables(hd, 128, 500000.0, device=DEV)
    y = native_lib.rope(x, cos[:s].contiguous(), sin[:s].contiguous(), 4, inverse=False)
    want = torch.cat([ref.apply_rope(x[:, :, :4].float(), cos[:s], sin[:s]), x[:, :, 4:].float()], dim=2)
    _close(y, want)
    back = native_lib.rope(y, cos[:s].contiguous(), sin[:s].contiguous(), 4, inverse=True)
    _close(back, x, rtol=3e-2, atol=3e-2)


def test_swiglu(native_lib):
    rows, h = 129, 1408
    gu = _rand(rows, 2 * h)
    guf = gu.float().requires_grad_(True)
    want = torch.nn.functional.silu(guf[:, :h]) * guf[:, h:]
    got = native_lib.swiglu_fwd(gu)
    _close(got, want)
    dh = _rand(rows, h)
    want.backward(dh.float())
    _close(native_lib.swiglu_bwd(dh, gu), guf.grad)


def test_embedding(native_lib):
    v, d, t = 1000, 256, 777
    table = _rand(v, d)
    ids = torch.randint(0, v, (t,), device=DEV)
    out = native_lib.embedding_fwd(ids, table)
    assert torch.equal(out, table[ids])
    dy = _rand(t, d, scale=0.1)
    dt = torch.empty_like(table)
    native_lib.embedding_bwd(dy, ids, dt, accumulate=False)
    want = torch.zeros(v, d, device=DEV).index_add_(0, ids, dy.float())
    _close(dt, want, rtol=5e-2, atol=2e-2)


@pytest.mark.parametrize("v", [1024, 128256, 1003])
def test_cross_entropy_fwd_bwd(native_lib, v):
    rows = 64
    ld = (v + 7) // 8 * 8
    buf = _rand(rows, ld, scale=2.0)
    logits = buf[:, :v]
    labels = torch.randint(0, v, (rows,), device=DEV)
    labels[::7] = -100
    lf = logits.float().clone().requires_grad_(True)
    z_w = 1e-3
    n = (labels != -100).sum().float()
    lse = torch.logsumexp(lf, -1)
    valid = labels != -100
    nll = (lse - lf.gather(1, labels.clamp_min(0)[:, None]).squeeze(1))[valid].sum()
    z = (lse[valid] ** 2).sum()
    ((nll + z_w * z) / n).backward()
    stats = torch.zeros(2, device=DEV)
    inv_n = (1.0 / n).reshape(1)
    native_lib.ce_fwd_bwd(logits, labels, stats, inv_n, z_w)
    _close(stats[0], nll.detach(), rtol=1e-3, atol=1e-3)
    _close(stats[1], z.detach(), rtol=1e-3, atol=1e-3)
    got, want = logits.float(), lf.grad
    assert (got - want).abs().max().item() < 2e-2 * want.abs().max().item() + 1e-6


@pytest.mark.parametrize("dtypes", [(torch.bfloat16, torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32, torch.float32)])
def test_adamw_matches_torch(native_lib, dtypes):
    torch.manual_seed(0)
    pd, gd, sd = dtypes
    n, n_decay = 10007, 6000
    p0 = torch.randn(n, device=DEV)
    p = p0.to(pd).clone()
    m = torch.zeros(n, device=DEV, dtype=sd)
    v = torch.zeros(n, device=DEV, dtype=sd)
    ref_p = torch.nn.Parameter(p.float().clone())
    opt = torch.optim.AdamW(
        [{"params": [ref_p], "weight_decay": 0.0}], lr=1e-2, betas=(0.9, 0.95), eps=1e-8
    )
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(gd)
        # reference: decay only the first n_decay elements
        with torch.no_grad():
            ref_p[:n_decay].mul_(1 - 1e-2 * 0.1)
        ref_p.grad = g.float()
        opt.step()
        native_lib.adamw_flat(p, g, m, v, n_decay, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
    # bf16 storage rounds parameters (|p| up to ~4 -> half an ulp is 0.016) and both moments every step
    tol = 6e-2 if pd == torch.bfloat16 else 1e-5
    assert (p.float() - ref_p.detach()).abs().max().item() < tol


def test_sumsq(native_lib):
    x = _rand(1 << 20)
    out = torch.zeros(1, device=DEV)
    native_lib.sumsq(x, out)
    _close(out[0], (x.float() ** 2).sum(), rtol=1e-4, atol=1e-4)


def test_bounded_wait_reports_status(native_lib):
    """A flag that nothing raises must end in a status code, not a hang (host reads it afterwards)."""
    fn = native_lib.lib().kf_test_flag_timeout  # argtypes are declared by the binding (pointer is 64-bit)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    native_lib.clear_status()
    fn(flag.data_ptr(), 1, 2_000_000)  # ~1 ms budget
    torch.cuda.synchronize()
    assert native_lib.read_status() == 6
    native_lib.clear_status()
    # the context is still healthy
    assert torch.ones(4, device=DEV).sum().item() == 4


def test_model_step_native_vs_reference(native_lib):
    from kempnerforge_b200.config import ModelConfig
    from kempnerforge_b200.models import Transformer
    from kempnerforge_b200.ops import functional as F

    torch.manual_seed(0)
    cfg = ModelConfig(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=1024, max_seq_len=128)
    model = Transformer(cfg).to(device=DEV, dtype=torch.bfloat16)
    tok = torch.randint(0, 1024, (2, 129), device=DEV)
    loss = model.compute_loss(tok[:, :-1], tok[:, 1:])
    loss.backward()
    g_native = {n: p.grad.float().clone() for n, p in model.named_parameters()}
    model.zero_grad()
    with F.force_reference():
        loss_ref = model.compute_loss(tok[:, :-1], tok[:, 1:])
        loss_ref.backward()
    assert abs(loss.item() - loss_ref.item()) < 5e-2
    for n, p in model.named_parameters():
        a, b = g_native[n], p.grad.float()
        denom = b.abs().max().item() + 1e-6
        assert (a - b).abs().max().item() / denom < 0.1, n


@pytest.mark.parametrize("ac", ["none", "full"])
def test_fused_dense_block_matches_op_by_op_path(native_lib, ac):
    """The hand-written block backward must agree with autograd over the individual native ops."""
    import kempnerforge_b200.models.transformer as tmod
    from kempnerforge_b200.config import ModelConfig
    from kempnerforge_b200.models import Transformer
    from kempnerforge_b200.parallel.flat import flatten_model

    torch.manual_seed(0)
    cfg = ModelConfig(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=1024, max_seq_len=128)
    model = Transformer(cfg).to(device=DEV, dtype=torch.bfloat16)
    for blk in model.layers.values():
        blk.ac_mode = ac
    tok = torch.randint(0, 1024, (2, 129), device=DEV)
    results = {}
    for fused in (True, False):
        tmod._FUSED_BLOCK_OFF = not fused
        model.zero_grad()
        model.train()
        loss = model.compute_loss(tok[:, :-1], tok[:, 1:])
        loss.backward()
        results[fused] = (loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters()})
    tmod._FUSED_BLOCK_OFF = False
    assert abs(results[True][0] - results[False][0]) < 2e-2
    for n, g in results[False][1].items():
        denom = g.abs().max().item() + 1e-6
        assert (results[True][1][n] - g).abs().max().item() / denom < 0.05, n
    # with flat gradient buffers the weight gradients land in the flat views
    flatten_model(model)
    model.zero_grad()
    for p in model.parameters():
        p.grad = None
    model.compute_loss(tok[:, :-1], tok[:, 1:]).backward()
    for g in model._kf_flat_groups:
        g.finalize_grads()
    for n, p in model.named_parameters():
        ref = results[False][1][n]
        assert (p.grad.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6) < 0.05, n


@pytest.mark.parametrize("ac", ["none", "full"])
def test_fused_attention_sublayer_of_moe_blocks_matches_op_by_op_path(native_lib, ac, monkeypatch):
    """Mixture-of-experts blocks run their attention sub-layer (norm, QKV + rotary, attention, O + residual) as one
    autograd node; losses and every gradient must agree with the op-by-op path, with and without activation
    checkpointing around the block, and with gradients deposited into flat buffers."""
    from kempnerforge_b200.config import ModelConfig
    from kempnerforge_b200.models import Transformer
    from kempnerforge_b200.ops import fused_block
    from kempnerforge_b200.parallel.flat import flatten_model

    torch.manual_seed(0)
    cfg = ModelConfig(dim=512, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=1024, max_seq_len=256, ffn_hidden_dim=1024,
                      num_experts=4, moe_top_k=2, moe_packed_experts=True)
    model = Transformer(cfg).to(device=DEV, dtype=torch.bfloat16)
    for blk in model.layers.values():
        blk.ac_mode = ac
    tok = torch.randint(0, 1024, (2, 257), device=DEV)
    calls = {"n": 0}
    real = fused_block.attn_half

    def counted(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    monkeypatch.setattr(fused_block, "attn_half", counted)
    results = {}
    for fused in (True, False):
        if fused:
            monkeypatch.delenv("KF_DISABLE_FUSED_ATTN_HALF", raising=False)
        else:
            monkeypatch.setenv("KF_DISABLE_FUSED_ATTN_HALF", "1")
        model.zero_grad()
        model.train()
        before = calls["n"]
        loss = model.compute_loss(tok[:, :-1], tok[:, 1:])
        loss.backward()
        assert (calls["n"] > before) == fused
        results[fused] = (loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None})
    assert native_lib.read_status() == 0
    assert abs(results[True][0] - results[False][0]) < 2e-2
    assert results[True][1].keys() == results[False][1].keys()
    # relative to the norm: a token whose top-k choice flips under bf16 noise changes single rows, not the whole gradient
    for n, g in results[False][1].items():
        assert ((results[True][1][n] - g).norm() / (g.norm() + 1e-12)).item() < 0.1, n   # norm-weight gradients are sums with heavy cancellation
    monkeypatch.delenv("KF_DISABLE_FUSED_ATTN_HALF", raising=False)
    flatten_model(model)
    for p in model.parameters():
        p.grad = None
    model.compute_loss(tok[:, :-1], tok[:, 1:]).backward()
    for g in model._kf_flat_groups:
        g.finalize_grads()
    for n, p in model.named_parameters():
        if n in results[False][1]:
            ref = results[False][1][n]
            assert ((p.grad.float() - ref).norm() / (ref.norm() + 1e-12)).item() < 0.1, n


# --------------------------------------------------------------------------- attention (tcgen05)
def _attn_inputs(b, s, h, hkv, hd, fused=True, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if fused:  # strided views of one projection output, as the model produces them
        qkv = torch.randn(b, s, h + 2 * hkv, hd, device="cuda", dtype=torch.bfloat16, generator=g)
        return qkv[:, :, :h], qkv[:, :, h:h + hkv], qkv[:, :, h + hkv:]
    mk = lambda n: torch.randn(b, s, n, hd, device="cuda", dtype=torch.bfloat16, generator=g)  # noqa: E731
    return mk(h), mk(hkv), mk(hkv)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(2, 256, 4, 2, 64), (1, 384, 4, 1, 128), (2, 200, 2, 2, 128), (1, 1000, 8, 2, 64),
                                   (1, 2048, 2, 1, 128)])
def test_attention_forward_matches_fp32_reference(native_lib, shape, causal):
    from kempnerforge_b200.ops import ref

    b, s, h, hkv, hd = shape
    q, k, v = _attn_inputs(b, s, h, hkv, hd)
    assert native_lib.attn_supported(q, k, v, causal)
    scale = 1.0 / math.sqrt(hd)
    out, lse = native_lib.attn_fwd(q, k, v, causal, None, scale)
    want = ref.attention(q.float(), k.float(), v.float(), causal=causal, scale=scale)
    assert native_lib.read_status() == 0
    err = (out.float() - want).abs().max().item()
    assert err < 2e-2, err
    # log-sum-exp of the scaled scores, natural log
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float().repeat_interleave(h // hkv, dim=2)) * scale
    if causal:
        scores = scores.masked_fill(~torch.ones(s, s, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    assert (lse - torch.logsumexp(scores, dim=-1)).abs().max().item() < 2e-2


def test_attention_forward_document_mask(native_lib):
    from kempnerforge_b200.ops import ref

    b, s, h, hkv, hd = 2, 512, 4, 2, 128
    q, k, v = _attn_inputs(b, s, h, hkv, hd, fused=False, seed=3)
    cuts = torch.tensor([[0, 100, 130, 400], [0, 256, 300, 301]], device="cuda")
    pos = torch.arange(s, device="cuda")
    doc = (pos[None, :, None] >= cuts[:, None, :]).sum(-1).to(torch.int32)
    out, _ = native_lib.attn_fwd(q, k, v, True, doc, 1.0 / math.sqrt(hd))
    want = ref.attention(q.float(), k.float(), v.float(), causal=True, doc_ids=doc)
    assert native_lib.read_status() == 0
    assert (out.float() - want).abs().max().item() < 2e-2


def test_attention_forward_large_scores_rescale(native_lib):
    """Row maxima that keep growing along the sequence exercise the lazy O rescaling."""
    from kempnerforge_b200.ops import ref

    b, s, h, hkv, hd = 1, 1024, 2, 2, 64
    q, k, v = _attn_inputs(b, s, h, hkv, hd, fused=False, seed=5)
    ramp = torch.linspace(0.2, 6.0, s, device="cuda")[None, :, None, None]
    k = (k.float() * ramp).to(torch.bfloat16)
    q = (q.float() * 2.0).to(torch.bfloat16)
    out, _ = native_lib.attn_fwd(q, k, v, True, None, 1.0 / math.sqrt(hd))
    want = ref.attention(q.float(), k.float(), v.float(), causal=True)
    assert native_lib.read_status() == 0
    assert (out.float() - want).abs().max().item() < 3e-2


# --------------------------------------------------------------------------- fp8 (tcgen05 kind::f8f6f4)
@pytest.mark.parametrize("e5m2", [False, True])
@pytest.mark.parametrize("shape", [(128, 256), (300, 520), (64, 4096)])
def test_fp8_scale_and_cast_match_torch(native_lib, shape, e5m2):
    rows, cols = shape
    x = _rand(rows, cols, scale=3.0)
    scale = native_lib.fp8_scale(x, e5m2)
    fmax = 57344.0 if e5m2 else 448.0
    assert abs(scale.item() - fmax / x.float().abs().max().item()) < 1e-3 * scale.item()
    row, t = native_lib.fp8_cast(x, scale, e5m2, True, True)
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    want = (x.float() * scale).clamp(-fmax, fmax).to(dt)
    assert torch.equal(row.view(dt).float(), want.float())
    assert torch.equal(t.view(dt).float(), want.float().t())


@pytest.mark.parametrize("fmt", [(False, False), (True, False)])
@pytest.mark.parametrize("shape", [(128, 256, 128), (384, 272, 400), (1024, 1024, 2048), (8192, 512, 4096)])
def test_fp8_gemm_matches_dequantised_reference(native_lib, shape, fmt):
    m, n, k = shape
    a, b = _rand(m, k), _rand(n, k, scale=0.05)
    sa, sb = native_lib.fp8_scale(a, fmt[0]), native_lib.fp8_scale(b, fmt[1])
    a8, _ = native_lib.fp8_cast(a, sa, fmt[0])
    b8, _ = native_lib.fp8_cast(b, sb, fmt[1])
    got = native_lib.gemm_fp8(a8, b8, sa, sb, fmt[0], fmt[1])
    dta = torch.float8_e5m2 if fmt[0] else torch.float8_e4m3fn
    dtb = torch.float8_e5m2 if fmt[1] else torch.float8_e4m3fn
    want = (a8.view(dta).float() @ b8.view(dtb).float().t()) / (sa * sb)
    assert native_lib.read_status() == 0
    _close(got, want, rtol=1e-2, atol=1e-2)
    acc = got.clone()
    native_lib.gemm_fp8(a8, b8, sa, sb, fmt[0], fmt[1], out=acc, accumulate=True)
    _close(acc, 2 * want, rtol=2e-2, atol=2e-2)


def test_fp8_linear_forward_backward_close_to_bf16(native_lib):
    from kempnerforge_b200.ops import functional as F

    torch.manual_seed(0)
    x = _rand(4, 128, 512).requires_grad_(True)
    w1 = (_rand(768, 512, scale=0.04)).requires_grad_(True)
    w2 = (_rand(256, 512, scale=0.04)).requires_grad_(True)
    g = _rand(4, 128, 1024)
    ref_y = torch.cat([x @ w1.t(), x @ w2.t()], dim=-1)
    ref_y.backward(g)
    want = [ref_y.detach(), x.grad.clone(), w1.grad.clone(), w2.grad.clone()]
    x.grad = w1.grad = w2.grad = None
    w1._kf_fp8 = w2._kf_fp8 = True
    y = F.fused_linear(x, [w1, w2])
    y.backward(g)
    assert native_lib.read_status() == 0
    for got, ref_t in zip([y.detach(), x.grad, w1.grad, w2.grad], want):
        rel = (got.float() - ref_t.float()).norm() / ref_t.float().norm()
        assert rel < 0.08, rel.item()


def _attn_reference_grads(q, k, v, dout, causal, doc=None):
    from kempnerforge_b200.ops import ref

    qf, kf_, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    out = ref.attention(qf, kf_, vf, causal=causal, doc_ids=doc)
    out.backward(dout.float())
    return out.detach(), qf.grad, kf_.grad, vf.grad


@pytest.fixture(params=[0, 1], ids=["dq_red", "dq_bulk_reduce"])
def dq_mode(native_lib, request):
    """Both ways the backward kernel accumulates dQ: per-element reductions and one bulk tensor reduction per tile."""
    prev = native_lib.attn_bwd_dq_mode(request.param)
    yield request.param
    native_lib.attn_bwd_dq_mode(prev)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(1, 128, 1, 1), (2, 256, 4, 2), (1, 384, 4, 1), (2, 200, 2, 2), (1, 1024, 8, 2)])
def test_attention_backward_matches_fp32_reference(native_lib, shape, causal, dq_mode):
    b, s, h, hkv = shape
    hd = 128
    q, k, v = _attn_inputs(b, s, h, hkv, hd, seed=11)
    dout = _rand(b, s, h, hd)
    scale = 1.0 / math.sqrt(hd)
    out, lse = native_lib.attn_fwd(q, k, v, causal, None, scale)
    dq, dk, dv = native_lib.attn_bwd(dout, q, k, v, out, lse, causal, None, scale)
    assert native_lib.read_status() == 0
    _, rq, rk, rv = _attn_reference_grads(q, k, v, dout, causal)
    for name, got, want in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        rel = (got.float() - want).norm() / want.norm()
        assert rel < 2e-2, (name, rel.item())


def test_attention_backward_document_mask_into_fused_gradient(native_lib, dq_mode):
    b, s, h, hkv, hd = 2, 512, 4, 2, 128
    q, k, v = _attn_inputs(b, s, h, hkv, hd, seed=13)
    cuts = torch.tensor([[0, 100, 130, 400], [0, 256, 300, 301]], device="cuda")
    doc = (torch.arange(s, device="cuda")[None, :, None] >= cuts[:, None, :]).sum(-1).to(torch.int32)
    dout = _rand(b, s, h, hd)
    scale = 1.0 / math.sqrt(hd)
    out, lse = native_lib.attn_fwd(q, k, v, True, doc, scale)
    dqkv = torch.zeros(b, s, h + 2 * hkv, hd, device="cuda", dtype=torch.bfloat16)
    native_lib.attn_bwd(dout, q, k, v, out, lse, True, doc, scale, dq=dqkv[:, :, :h], dk=dqkv[:, :, h:h + hkv],
                        dv=dqkv[:, :, h + hkv:])
    assert native_lib.read_status() == 0
    _, rq, rk, rv = _attn_reference_grads(q, k, v, dout, True, doc)
    want = torch.cat([rq, rk, rv], dim=2)
    rel = (dqkv.float() - want).norm() / want.norm()
    assert rel < 2e-2, rel.item()


def test_attention_autograd_function_native_policy(native_lib, monkeypatch):
    from kempnerforge_b200.ops import functional as F

    monkeypatch.setenv("KF_ATTN", "native")
    b, s, h, hkv, hd = 1, 256, 4, 2, 128
    q, k, v = (t.clone().requires_grad_(True) for t in _attn_inputs(b, s, h, hkv, hd, fused=False, seed=17))
    dout = _rand(b, s, h, hd)
    out = F.attention(q, k, v, causal=True)
    out.backward(dout)
    _, rq, rk, rv = _attn_reference_grads(q, k, v, dout, True)
    for got, want in ((q.grad, rq), (k.grad, rk), (v.grad, rv)):
        assert ((got.float() - want).norm() / want.norm()) < 2e-2


# --------------------------------------------------------------------------- ragged grouped GEMM (MoE experts)
@pytest.fixture(params=["pair", "single"])
def grouped_tiles(request, native_lib):
    """Runs a grouped-GEMM test on both tilings: CTA pairs (256-row tiles, the default) and single-CTA 128 x 256."""
    native_lib.grouped_pair_mode(1 if request.param == "pair" else 0)
    yield request.param
    native_lib.grouped_pair_mode(1)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("counts", [[128, 128, 128, 128], [5, 0, 300, 77, 130, 1], [1000, 24], [0, 0, 513]])
def test_grouped_gemm_forward_backward(native_lib, counts, layout, grouped_tiles):
    from kempnerforge_b200.ops import grouped

    torch.manual_seed(0)
    e, k, n = len(counts), 192, 320
    rows = sum(counts)
    x = _rand(rows, k).requires_grad_(True)
    w = (_rand(e, k, n, scale=0.05) if layout == "kn" else _rand(e, n, k, scale=0.05)).requires_grad_(True)
    cnt = torch.tensor(counts, device="cuda")
    y = grouped.grouped_linear(x, w, cnt, layout)
    g = _rand(rows, n)
    y.backward(g)
    assert native_lib.read_status() == 0
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    outs, start = [], 0
    for i, c in enumerate(counts):
        we = wf[i] if layout == "kn" else wf[i].t()
        outs.append(xf[start:start + c] @ we)
        start += c
    want = torch.cat(outs)
    want.backward(g.float())
    _close(y, want)
    _close(x.grad, xf.grad)
    _close(w.grad, wf.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("counts", [[128, 128, 128, 128], [5, 0, 300, 77, 130, 1], [1000, 24], [0, 0, 513], [64, 63, 65], [449, 1, 15, 16, 17]])
def test_grouped_wgrad_matches_per_expert_products(native_lib, counts, grouped_tiles):
    """Ragged reduction ranges: rows of the next expert, and NaN rows past the last expert, must not leak in."""
    torch.manual_seed(0)
    m, n = 200, 328
    rows = sum(counts)
    pad = 70
    a = _rand(rows + pad, m)
    b = _rand(rows + pad, n)
    a[rows:] = float("nan")
    b[rows:] = float("nan")
    offsets = torch.zeros(len(counts) + 1, dtype=torch.int32, device="cuda")
    offsets[1:] = torch.tensor(counts, device="cuda").cumsum(0)
    got = native_lib.grouped_wgrad(a, b, offsets)
    assert native_lib.read_status() == 0
    start = 0
    for e, c in enumerate(counts):
        want = a[start:start + c].float().t() @ b[start:start + c].float()
        _close(got[e], want, rtol=3e-2, atol=3e-2)
        start += c


# --------------------------------------------------------------------------- Newton-Schulz on the tensor cores
@pytest.mark.parametrize("shape", [(256, 256), (128, 512), (512, 128), (1024, 384), (64, 4096)])
def test_newton_schulz_matches_the_fp32_formulation_for_wide_and_tall_matrices(native_lib, shape):
    from kempnerforge_b200.ops import ref
    from kempnerforge_b200.training.optimizer import newton_schulz

    torch.manual_seed(0)
    g = torch.randn(*shape, device="cuda")
    got = newton_schulz(g, 5)
    want = ref.newton_schulz(g, 5)          # un-transposed fp32 reference (Gram on the row side)
    assert got.shape == want.shape and got.dtype == torch.float32 and native_lib.read_status() == 0
    rel = ((got - want).norm() / want.norm()).item()
    assert rel < 3e-2, rel
    sv = torch.linalg.svdvals(got)
    assert sv.max() < 1.3
    if max(shape) >= 2 * min(shape):       # a random square matrix has singular values near zero that five steps cannot lift
        assert sv.min() > 0.3


# --------------------------------------------------------------------------- memory safety without a sanitizer
_SENTINEL = 12288.0  # exactly representable in bf16


def _guarded(shape, dtype=torch.bfloat16, pad=4096):
    """A tensor of ``shape`` carved out of a larger buffer whose margins hold a sentinel value."""
    n = 1
    for d in shape:
        n *= d
    flat = torch.full((n + 2 * pad,), _SENTINEL, dtype=dtype, device="cuda")
    return flat, flat[pad:pad + n].view(*shape)


def _margins_intact(flat, n, pad=4096):
    return bool((flat[:pad] == _SENTINEL).all()) and bool((flat[pad + n:] == _SENTINEL).all())


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (130, 264, 72), (257, 520, 200), (1000, 136, 4096)])
def test_gemm_ragged_shapes_stay_inside_their_output_and_repeat_bit_exactly(native_lib, mode, m, n, k):
    torch.manual_seed(0)
    a, b = _rand(m, k), _rand(n, k)
    flat, out = _guarded((m, n))
    native_lib.gemm(a, b, out=out, mode=mode)
    assert native_lib.read_status() == 0 and _margins_intact(flat, m * n)
    _close(out, a.float() @ b.float().t())
    again = native_lib.gemm(a, b, mode=mode)
    assert torch.equal(out, again)            # fixed reduction order: a difference would mean a race


@pytest.mark.parametrize("counts", [[5, 0, 300, 77, 130, 1], [0, 0, 513], [1], [257, 255, 0, 700]])
def test_grouped_kernels_stay_inside_their_outputs_and_repeat_bit_exactly(native_lib, counts, grouped_tiles):
    torch.manual_seed(0)
    e, k, n = len(counts), 192, 328
    rows = sum(counts)
    x, w, g = _rand(rows, k), _rand(e, n, k, scale=0.05), _rand(rows, n)
    offsets = torch.zeros(e + 1, dtype=torch.int32, device="cuda")
    offsets[1:] = torch.tensor(counts, device="cuda").cumsum(0)
    flat_y, y = _guarded((rows, n))
    native_lib.grouped_gemm(x, w, offsets, b_mn=False, out=y)
    flat_w, dw = _guarded((e, n, k))
    native_lib.grouped_wgrad(g, x, offsets, out=dw)
    assert native_lib.read_status() == 0
    assert _margins_intact(flat_y, rows * n) and _margins_intact(flat_w, e * n * k)
    assert torch.equal(y, native_lib.grouped_gemm(x, w, offsets, b_mn=False))
    assert torch.equal(dw, native_lib.grouped_wgrad(g, x, offsets))
    assert not torch.isnan(dw.float()).any() and not (dw == _SENTINEL).any()


def test_row_kernels_stay_inside_their_outputs_and_repeat_bit_exactly(native_lib):
    torch.manual_seed(0)
    rows, d = 1003, 4096
    x, w, dy = _rand(rows, d), _rand(d), _rand(rows, d)
    y, rstd = native_lib.rmsnorm_fwd(x, w, 1e-5)
    y2, rstd2 = native_lib.rmsnorm_fwd(x, w, 1e-5)
    assert torch.equal(y, y2) and torch.equal(rstd, rstd2)
    flat, dx = _guarded((rows, d))
    dx1, dw1 = native_lib.rmsnorm_bwd(dy, x, w, rstd, out=dx)
    dx2, dw2 = native_lib.rmsnorm_bwd(dy, x, w, rstd)
    assert _margins_intact(flat, rows * d) and native_lib.read_status() == 0
    assert torch.equal(dw1, dw2) and torch.equal(dx1, dx2)
    gu = _rand(rows, 2 * 1408)
    assert torch.equal(native_lib.swiglu_fwd(gu), native_lib.swiglu_fwd(gu))


def test_attention_forward_repeats_bit_exactly(native_lib):
    torch.manual_seed(0)
    q, k, v = _rand(1, 384, 8, 128), _rand(1, 384, 2, 128), _rand(1, 384, 2, 128)
    o1, l1 = native_lib.attn_fwd(q, k, v, True, None, 128 ** -0.5)
    o2, l2 = native_lib.attn_fwd(q, k, v, True, None, 128 ** -0.5)
    assert torch.equal(o1, o2) and torch.equal(l1, l2) and native_lib.read_status() == 0


# --------------------------------------------------------------------------- MoE routing / sort / gather / combine
@pytest.mark.parametrize("sigmoid", [False, True])
@pytest.mark.parametrize("shape", [(64, 8, 2), (1000, 64, 6), (333, 160, 8)])
def test_router_topk_matches_torch(native_lib, shape, sigmoid):
    from kempnerforge_b200.ops import moe_ops

    t, e, k = shape
    torch.manual_seed(1)
    logits = (torch.randn(t, e, device="cuda") * 2).requires_grad_(True)
    bias = (torch.randn(e, device="cuda") * 0.1) if sigmoid else None
    w, idx, counts, mean, z = moe_ops.route(logits, bias, sigmoid, k)
    lf = logits.detach().clone().requires_grad_(True)
    scores = torch.sigmoid(lf + bias) if sigmoid else torch.softmax(lf, dim=-1)
    rw, ridx = torch.topk(scores, k, dim=-1)
    rw = rw / rw.sum(-1, keepdim=True)
    assert torch.equal(idx.sort(dim=1).values, ridx.sort(dim=1).values)
    assert torch.equal(idx, ridx)
    assert torch.allclose(w, rw, atol=1e-5)
    assert torch.equal(counts, torch.bincount(ridx.reshape(-1), minlength=e).float())
    assert torch.allclose(mean, scores.mean(0), atol=1e-5)
    rz = torch.logsumexp(lf, dim=-1).pow(2).mean()
    assert torch.allclose(z, rz, rtol=1e-4)
    gw = torch.randn_like(w)
    gm = torch.randn(e, device="cuda")
    (w * gw).sum().add((mean * gm).sum()).add(z * 0.3).backward()
    (rw * gw).sum().add((scores.mean(0) * gm).sum()).add(rz * 0.3).backward()
    assert torch.allclose(logits.grad, lf.grad, atol=2e-5, rtol=1e-3)


def test_moe_sort_gather_combine_match_torch(native_lib):
    from kempnerforge_b200.ops import moe_ops

    torch.manual_seed(2)
    t, e, k, d = 777, 16, 4, 256
    idx = torch.stack([torch.randperm(e, device="cuda")[:k] for _ in range(t)])
    offsets, row_of_slot, slot_of_row = moe_ops.sort_by_expert(idx, e)
    order = torch.argsort(idx.reshape(-1), stable=True)
    assert torch.equal(slot_of_row.long(), order)
    assert torch.equal(offsets[1:].long(), torch.bincount(idx.reshape(-1), minlength=e).cumsum(0))
    x = _rand(t, d).requires_grad_(True)
    w = torch.rand(t, k, device="cuda").to(torch.bfloat16).requires_grad_(True)
    xs = moe_ops.gather_rows(x, slot_of_row, row_of_slot, k)
    assert torch.equal(xs, x.detach()[order // k])
    y = (xs.float() * 1.5).to(torch.bfloat16)          # stand-in for the expert computation, keeps the graph
    out = moe_ops.combine_rows(y, w, row_of_slot, slot_of_row)
    g = _rand(t, d)
    out.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = (xr[order // k] * 1.5).to(torch.bfloat16).float()
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device="cuda")
    want = (yr[inv].view(t, k, d) * wr[:, :, None]).sum(1)
    want.backward(g.float())
    _close(out, want)
    _close(x.grad, xr.grad, rtol=3e-2, atol=3e-2)
    _close(w.grad, wr.grad, rtol=3e-2, atol=3e-2)


def test_moe_layer_native_matches_reference_path(native_lib):
    from kempnerforge_b200.models.moe import build_moe
    from kempnerforge_b200.ops import functional as F

    torch.manual_seed(3)
    layer = build_moe(256, 512, 8, 2, packed_experts=True).to(device="cuda", dtype=torch.bfloat16)
    x = _rand(2, 192, 256)
    xa = x.clone().requires_grad_(True)
    ya = layer(xa)
    ya.float().sum().backward()
    ga = {n: p.grad.clone() for n, p in layer.named_parameters() if p.grad is not None}
    layer.zero_grad()
    with F.force_reference():
        xb = x.clone().requires_grad_(True)
        yb = layer(xb)
        yb.float().sum().backward()
    assert native_lib.read_status() == 0
    _close(ya, yb, rtol=3e-2, atol=3e-2)
    _close(xa.grad, xb.grad, rtol=5e-2, atol=5e-2)
    for n, p in layer.named_parameters():
        if p.grad is not None and n in ga:
            _close(ga[n], p.grad, rtol=6e-2, atol=6e-2)


# --------------------------------------------------------------------------- end-to-end variants on one GPU
def _tiny_job(**over):
    from kempnerforge_b200.config import config_from_dict

    cfg = {
        "model": dict(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=512, ffn_hidden_dim=512, max_seq_len=128),
        "train": dict(batch_size=4, seq_len=128, max_steps=20, mixed_precision="bf16", seed=0),
        "optimizer": dict(lr=2e-3), "scheduler": dict(name="constant", warmup_steps=0),
        "metrics": dict(log_interval=1000),
    }
    for section, vals in over.items():
        cfg.setdefault(section, {}).update(vals)
    return config_from_dict(cfg)


def _overfit(trainer, steps=12):
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 512, (4, 129), generator=g)
    batch = {"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}
    return [trainer.train_step([batch])["loss"] for _ in range(steps)]


def test_fp8_training_learns(native_lib):
    from kempnerforge_b200.ops import fp8
    from kempnerforge_b200.training.trainer import Trainer

    t = Trainer(_tiny_job(train=dict(mixed_precision="fp8")), init_dist=False)
    tagged = [n for n, p in t.model.named_parameters() if fp8.is_fp8_weight(p)]
    assert any("q_proj" in n for n in tagged) and any("down_proj" in n for n in tagged)
    assert not any("output_head" in n or "embedding" in n for n in tagged)
    losses = _overfit(t)
    assert native_lib.read_status() == 0
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 1.0, losses


@pytest.mark.parametrize("router", ["softmax_topk", "sigmoid_topk"])
def test_moe_training_learns_on_native_kernels(native_lib, router):
    from kempnerforge_b200.training.trainer import Trainer

    t = Trainer(_tiny_job(model=dict(num_experts=4, moe_top_k=2, moe_router=router, moe_packed_experts=True)),
                init_dist=False)
    losses = _overfit(t)
    assert native_lib.read_status() == 0
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 1.0, losses


def test_native_attention_policy_in_training(native_lib, monkeypatch):
    """KF_ATTN=native: the tcgen05 attention kernels (forward and backward) inside the fused block train a model."""
    from kempnerforge_b200.training.trainer import Trainer

    monkeypatch.setenv("KF_ATTN", "native")
    cfg = _tiny_job(model=dict(dim=512, n_heads=4, n_kv_heads=2, ffn_hidden_dim=1024),
                    train=dict(activation_checkpointing="full"))
    t = Trainer(cfg, init_dist=False)
    losses = _overfit(t)
    assert native_lib.read_status() == 0
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 1.0, losses


@pytest.mark.parametrize("opt_name", ["adamw", "lion"])
def test_a_hand_written_loop_on_the_gpu_trains_like_the_trainer(native_lib, opt_name):
    """``loss.backward(); clip_grad_norm_(); optimizer.step(); optimizer.zero_grad()`` over ``build_parallel_model`` /
    ``build_optimizer`` with no engine call: the optimizer hooks reduce, scale and publish, so the losses are the
    trainer's (same kernels in the same order; the fused head + loss of the trainer against logits + loss here)."""
    from kempnerforge_b200.distributed import build_parallel_model, clip_grad_norm_
    from kempnerforge_b200.training.loss import build_loss_fn
    from kempnerforge_b200.training.optimizer import build_optimizer
    from kempnerforge_b200.training.trainer import Trainer

    cfg = _tiny_job(optimizer=dict(name=opt_name, lr=2e-3 if opt_name == "adamw" else 2e-4), train=dict(grad_clip_norm=1.0))
    t = Trainer(cfg, init_dist=False)
    init = {n: p.detach().clone() for n, p in t.model.named_parameters()}
    want = _overfit(t, steps=8)
    model = build_parallel_model(cfg.model, torch.device("cuda"), None, param_dtype=cfg.train.param_dtype)
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(init[n])
    opt, loss_fn = build_optimizer(model, cfg.optimizer), build_loss_fn(cfg.train)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 512, (4, 129), generator=g).cuda()
    ids, labels = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    got = []
    for _ in range(8):
        loss = loss_fn(model(ids), labels)
        loss.backward()
        # gradients that fused nodes wrote into the flat buffers are visible as ``.grad`` once backward has returned
        missing = [n for n, p in model.named_parameters() if p.requires_grad and p.grad is None]
        assert not missing, missing
        assert all(bool(torch.isfinite(p.grad.float()).all()) for p in model.parameters())
        clip_grad_norm_(model, 1.0)
        opt.step()
        opt.zero_grad()
        got.append(float(loss.detach()))
    assert native_lib.read_status() == 0
    assert got[-1] < got[0] - 0.5, got
    for step, (a, b) in enumerate(zip(got, want)):
        assert abs(a - b) <= 0.05 * max(1.0, abs(b)), (step, got, want)


@pytest.mark.parametrize("name", ["lion", "schedule_free_adamw"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lion_and_schedule_free_kernels_match_python_rules(native_lib, name, dtype):
    """The fused update kernels against the same optimizers running their PyTorch formulas on the CPU."""
    from kempnerforge_b200.config import OptimizerConfig
    from kempnerforge_b200.training.optimizer import build_optimizer

    torch.manual_seed(0)
    ref_m = torch.nn.Linear(64, 96, bias=True).to(dtype)
    dev_m = torch.nn.Linear(64, 96, bias=True).to(dtype)
    dev_m.load_state_dict(ref_m.state_dict())
    dev_m = dev_m.cuda()
    cfg = OptimizerConfig(name=name, lr=1e-2, weight_decay=0.1)
    ro, do = build_optimizer(ref_m, cfg), build_optimizer(dev_m, cfg)
    for step in range(4):
        g = torch.Generator().manual_seed(step)
        for (pr, pd) in zip(ref_m.parameters(), dev_m.parameters()):
            grad = torch.randn(pr.shape, generator=g).to(dtype)
            pr.grad, pd.grad = grad.clone(), grad.cuda()
        ro.step()
        do.step()
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for pr, pd in zip(ref_m.parameters(), dev_m.parameters()):
        assert torch.allclose(pr.float(), pd.float().cpu(), atol=tol, rtol=tol), (pr.float() - pd.float().cpu()).abs().max()


@pytest.mark.parametrize("shape", [(256, 128, 64), (512, 384, 256), (1000, 1024, 520), (8192, 14336, 4096)])
def test_gemm_swiglu_epilogue_matches_two_kernel_path(native_lib, shape):
    m, f, k = shape
    x = _rand(m, k)
    w = _rand(2 * f, k, scale=0.05)
    assert native_lib.gemm_swiglu_supported(x, w)
    h, gu = native_lib.gemm_swiglu(x, w, want_gu=True)
    h_only, none = native_lib.gemm_swiglu(x, w, want_gu=False)
    assert none is None and native_lib.read_status() == 0
    gu_ref = native_lib.gemm(x, w)
    h_ref = native_lib.swiglu_fwd(gu_ref)
    _close(gu, gu_ref, rtol=1e-2, atol=1e-2)
    _close(h, h_ref, rtol=2e-2, atol=2e-2)
    assert torch.equal(h, h_only)
    want = torch.nn.functional.silu(x.float() @ w[:f].float().t()) * (x.float() @ w[f:].float().t())
    _close(h, want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(2, 256, 4, 2, 64), (1, 384, 4, 1, 128), (2, 200, 2, 2, 128), (1, 1000, 8, 2, 64)])
def test_attention_forward_single_tile_kernel(native_lib, monkeypatch, shape, causal):
    """The one-query-tile kernel (used for short sequences) on shapes that the two-tile kernel takes by default."""
    from kempnerforge_b200.ops import ref

    monkeypatch.setenv("KF_ATTN_FWD", "1")
    b, s, h, hkv, hd = shape
    q, k, v = _attn_inputs(b, s, h, hkv, hd, seed=23)
    out, _ = native_lib.attn_fwd(q, k, v, causal, None, 1.0 / math.sqrt(hd))
    want = ref.attention(q.float(), k.float(), v.float(), causal=causal)
    assert native_lib.read_status() == 0
    assert (out.float() - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("shape", [(2, 128, 4, 2, 128, 256), (1, 512, 8, 2, 128, 520), (2, 256, 4, 4, 64, 128)])
def test_gemm_rope_epilogue_matches_projection_then_rotation(native_lib, shape):
    """Fused Q | K | V projection with the rotary embedding in the GEMM epilogue against an fp32 product followed by
    the reference rotation; the V columns must come out un-rotated."""
    from kempnerforge_b200.ops import ref

    b, s, h, hkv, hd, k = shape
    n = (h + 2 * hkv) * hd
    x, w = _rand(b * s, k), _rand(n, k) * 0.1
    cos, sin = ref.rope_tables(hd, s, 500000.0, device=DEV)
    cos, sin = cos[:s].contiguous(), sin[:s].contiguous()
    got = native_lib.gemm(x, w, rope=(cos, sin, s, (h + hkv) * hd, hd), mode=2)
    assert native_lib.read_status() == 0
    full = (x.float() @ w.float().t()).view(b, s, h + 2 * hkv, hd)
    want = torch.cat([ref.apply_rope(full[:, :, : h + hkv], cos, sin), full[:, :, h + hkv:]], dim=2).reshape(b * s, n)
    _close(got, want, rtol=2e-2, atol=2e-2)
    plain = native_lib.gemm(x, w, mode=2)
    assert torch.equal(got.view(b, s, -1, hd)[:, :, h + hkv:], plain.view(b, s, -1, hd)[:, :, h + hkv:])


@pytest.mark.parametrize("shape", [(2, 256, 4, 2), (1, 384, 4, 1), (2, 200, 2, 2)])
def test_attention_backward_with_inverse_rotary_epilogue(native_lib, shape):
    """dq / dk through the inverse rotary embedding inside the backward (dq in its fp32 -> bf16 pass, dk in the kernel
    epilogue) against the plain backward followed by the separate inverse rotation; dv is unchanged."""
    from kempnerforge_b200.ops import ref

    b, s, h, hkv = shape
    hd = 128
    q, k, v = _attn_inputs(b, s, h, hkv, hd, seed=17)
    dout = _rand(b, s, h, hd)
    scale = 1.0 / math.sqrt(hd)
    cos, sin = ref.rope_tables(hd, s, 500000.0, device=DEV)
    cos, sin = cos[:s].contiguous(), sin[:s].contiguous()
    out, lse = native_lib.attn_fwd(q, k, v, True, None, scale)
    dqkv = torch.zeros(b, s, h + 2 * hkv, hd, device="cuda", dtype=torch.bfloat16)
    native_lib.attn_bwd(dout, q, k, v, out, lse, True, None, scale, dq=dqkv[:, :, :h], dk=dqkv[:, :, h:h + hkv],
                        dv=dqkv[:, :, h + hkv:], rope=(cos, sin))
    assert native_lib.read_status() == 0
    _, rq, rk, rv = _attn_reference_grads(q, k, v, dout, True)
    want = torch.cat([ref.apply_rope(rq, cos, -sin), ref.apply_rope(rk, cos, -sin), rv], dim=2)
    for name, lo, hi in (("dq", 0, h), ("dk", h, h + hkv), ("dv", h + hkv, h + 2 * hkv)):
        rel = (dqkv[:, :, lo:hi].float() - want[:, :, lo:hi]).norm() / want[:, :, lo:hi].norm()
        assert rel < 2e-2, (name, rel.item())


class _FakePeers:
    """Stands in for a symmetric-memory buffer: the 'ranks' are separate tensors on this one GPU, which is all the
    gathering kernels need (they only ever load from the pointers they are given and never wait for a peer)."""

    def __init__(self, tensors, rank):
        import ctypes

        self.tensors = tensors
        self.world, self.rank = len(tensors), rank
        ptrs = [t.data_ptr() for t in tensors] + [0] * (8 - len(tensors))
        self.peer_ptrs = (ctypes.c_longlong * 8)(*ptrs)
        self.multicast_ptr = None


def _shards_of(weights, world):
    """Per-rank shard buffers holding piece r of every weight, packed in order; returns (shards, shard offsets)."""
    offs, acc = [], 0
    for w in weights:
        offs.append(acc)
        acc += w.numel() // world
    shards = []
    for r in range(world):
        sh = torch.empty(acc, device=DEV, dtype=torch.bfloat16)
        for w, o in zip(weights, offs):
            piece = w.numel() // world
            sh[o:o + piece] = w.reshape(-1)[r * piece:(r + 1) * piece]
        shards.append(sh)
    return shards, offs


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 5)])
@pytest.mark.parametrize("epi", [0, 1, 2])
def test_gemm_with_gathered_weight_operand(native_lib, world, rank, epi):
    """The weight-gathering GEMM against the plain kernels on the assembled weight: plain (+ residual), SwiGLU and
    rotary epilogues; the staging buffer must hold the whole operand afterwards."""
    from kempnerforge_b200.ops import ref

    torch.manual_seed(world * 10 + rank)
    m, k = 512, 512
    if epi == 1:
        rows = [1024, 1024]          # gate, up
    elif epi == 2:
        rows = [1024, 256, 256]      # q, k, v (head dim 128: 8 / 2 / 2 heads)
    else:
        rows = [1024]
    weights = [_rand(r, k) * 0.1 for r in rows]
    x = _rand(m, k)
    shards, offs = _shards_of(weights, world)
    total_rows = sum(rows)
    stage = torch.full((total_rows * k,), float("nan"), device=DEV, dtype=torch.bfloat16)
    flags = torch.zeros(256, dtype=torch.int32, device=DEV)
    plan = {"symm": _FakePeers(shards, rank), "seg_rows": rows, "seg_src": offs, "stage": stage, "flags": flags}
    w_full = torch.cat(weights, dim=0)
    if epi == 0:
        res = _rand(m, total_rows)
        got = native_lib.gemm_gather(x, plan, total_rows, epi=0, residual=res)
        want = native_lib.gemm(x, w_full, residual=res, mode=2)
        assert torch.equal(got, want)
    elif epi == 1:
        h, gu = native_lib.gemm_gather(x, plan, rows[0], epi=1, want_gu=True)
        h2, gu2 = native_lib.gemm_swiglu(x, w_full, want_gu=True)
        assert torch.equal(h, h2) and torch.equal(gu, gu2)
    else:
        s, hd = 256, 128
        cos, sin = ref.rope_tables(hd, s, 500000.0, device=DEV)
        cos, sin = cos[:s].contiguous(), sin[:s].contiguous()
        rope = (cos, sin, s, rows[0] + rows[1], hd)
        got = native_lib.gemm_gather(x, plan, total_rows, epi=2, rope=rope)
        want = native_lib.gemm(x, w_full, rope=rope, mode=2)
        assert torch.equal(got, want)
    assert native_lib.read_status() == 0
    assert torch.equal(stage.view(total_rows, k), w_full)


def test_symm_pull_and_shard_reduce_scatter_kernels(native_lib):
    """Pull (all-gather of pieces into the full layout) and the reduce-scatter of full-layout gradients into the
    shard layout, with the ranks emulated as separate buffers on one GPU."""
    world = 4
    lens = [4096 * 8, 64 * world, 1024 * world]          # a matrix, a tiny vector, another tensor
    full_off, acc = [], 0
    for n in lens:
        full_off.append(acc)
        acc += n
    params = [_rand(n) for n in lens]
    shards, offs = _shards_of(params, world)
    dst = torch.zeros(acc, device=DEV, dtype=torch.bfloat16)
    native_lib.symm_pull(_FakePeers(shards, 1), full_off, lens, offs, dst)
    assert torch.equal(dst, torch.cat(params))
    # gradients: every "rank" has a full-layout buffer; rank r ends with the mean of its pieces
    grads = [_rand(acc) for _ in range(world)]
    mean = torch.stack([g.float() for g in grads]).mean(0)
    for rank in range(world):
        out = torch.zeros(acc // world, device=DEV, dtype=torch.bfloat16)
        native_lib.symm_rs_shard(_FakePeers(grads, rank), full_off, lens, offs, out, accumulate=False)
        want = torch.cat([mean[o + rank * (n // world): o + (rank + 1) * (n // world)] for o, n in zip(full_off, lens)])
        _close(out, want, rtol=1e-2, atol=1e-2)
        native_lib.symm_rs_shard(_FakePeers(grads, rank), full_off, lens, offs, out, accumulate=True)
        _close(out, 2 * want, rtol=2e-2, atol=2e-2)
    assert native_lib.read_status() == 0


@pytest.mark.parametrize("z_w", [0.0, 1e-3])
def test_vocab_parallel_cross_entropy_kernels_match_full_cross_entropy(native_lib, z_w):
    """Two vocabulary shards handled by the two-phase kernels (statistics -> exchange -> gradient in place), combined
    the way the ranks combine them, against the fp32 cross entropy over the whole vocabulary."""
    torch.manual_seed(3)
    t, v, tp = 300, 1024, 2
    vl = v // tp
    logits = (_rand(t, v) * 4).contiguous()
    labels = torch.randint(0, v, (t,), device=DEV)
    labels[::7] = -100
    shards = [logits[:, r * vl:(r + 1) * vl].contiguous() for r in range(tp)]
    stats = [native_lib.ce_vp_stats(s, labels, r * vl) for r, s in enumerate(shards)]
    gmax = torch.stack([s[0] for s in stats]).max(0).values
    sumexp = sum(s[1] * torch.exp(s[0] - gmax) for s in stats)
    picked = sum(s[2] for s in stats)
    lse = gmax + torch.log(sumexp)
    valid = labels != -100
    n = valid.sum().float()
    loss = (torch.where(valid, lse - picked, torch.zeros_like(lse)).sum() + z_w * torch.where(valid, lse * lse, torch.zeros_like(lse)).sum()) / n
    lf = logits.float().requires_grad_(True)
    lse_ref = torch.logsumexp(lf, -1)
    ref = torch.nn.functional.cross_entropy(lf, labels, ignore_index=-100) + z_w * (lse_ref[valid] ** 2).sum() / n
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    up = torch.full((1,), 0.5, device=DEV)
    for r, s in enumerate(shards):
        g = native_lib.ce_vp_bwd(s, labels, r * vl, lse, (1.0 / n).reshape(1), up, z_w)
        want = 0.5 * lf.grad[:, r * vl:(r + 1) * vl]
        assert (g.float() - want).abs().max() <= 2e-2 * want.abs().max() + 1e-6


@pytest.mark.parametrize("shape", [(1000, 2, 8, 1.0), (4096, 6, 64, 1.25), (77, 1, 4, 0.5)])
def test_moe_capacity_mask_kernel_matches_the_reference_rule(native_lib, shape):
    """First `cap` tokens in sequence order of every (slot, expert) pair keep their weight (the rule of the
    reference's Python loops), evaluated by one kernel."""
    import math

    from kempnerforge_b200.models.moe import apply_capacity

    t, k, e, cf = shape
    torch.manual_seed(t)
    idx = torch.randint(0, e, (t, k), device=DEV)
    w = torch.rand(t, k, device=DEV)
    got, _ = apply_capacity(w, idx, e, cf)
    cap = max(1, math.ceil(t * k / e * cf))
    want = w.clone().cpu()
    ic = idx.cpu()
    for j in range(k):
        for ex in range(e):
            rows = (ic[:, j] == ex).nonzero(as_tuple=True)[0]
            want[rows[cap:], j] = 0.0
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("layout", ["kn", "nk"])
@pytest.mark.parametrize("counts,extra", [([128, 128, 128, 128], 0), ([5, 0, 300, 77, 130, 1], 0), ([1000, 24], 200), ([0, 0, 513], 64)])
def test_grouped_expert_ffn_with_swiglu_epilogue(native_lib, counts, layout, extra, monkeypatch, grouped_tiles):
    """Expert feed-forward (gate / up grouped GEMM with the SwiGLU epilogue, ragged SwiGLU gradient, accumulating
    input-gradient GEMMs) against an fp32 per-expert reference.  ``extra`` rows beyond the last expert stand for a
    buffer sized by an upper bound: they must be ignored.  No row count may be read on the host."""
    from kempnerforge_b200.ops import grouped

    torch.manual_seed(1)
    e, d, f = len(counts), 192, 256
    rows = sum(counts)
    x = _rand(rows + extra, d)
    x[rows:] = float("nan")
    x.requires_grad_(True)
    shape_in, shape_out = ((e, d, f), (e, f, d)) if layout == "kn" else ((e, f, d), (e, d, f))
    wg, wu = (_rand(*shape_in, scale=0.05).requires_grad_(True) for _ in range(2))
    wd = _rand(*shape_out, scale=0.05).requires_grad_(True)
    cnt = torch.tensor(counts, device="cuda")
    off = grouped.offsets_of(cnt)

    def boom(*a, **k):
        raise AssertionError("host read inside the expert feed-forward")

    monkeypatch.setattr(torch.Tensor, "item", boom)
    monkeypatch.setattr(torch.Tensor, "tolist", boom)
    y = grouped.grouped_ffn(x, cnt, wg, wu, wd, layout, offsets=off)
    g = _rand(rows + extra, d)
    y.backward(g)
    monkeypatch.undo()
    assert native_lib.read_status() == 0
    xf = x.detach()[:rows].float().requires_grad_(True)
    wgf, wuf, wdf = (w.detach().float().requires_grad_(True) for w in (wg, wu, wd))
    outs, start = [], 0
    for i, c in enumerate(counts):
        t = (lambda w: w[i] if layout == "kn" else w[i].t())
        xe = xf[start:start + c]
        outs.append((torch.nn.functional.silu(xe @ t(wgf)) * (xe @ t(wuf))) @ t(wdf))
        start += c
    want = torch.cat(outs)
    want.backward(g[:rows].float())
    _close(y[:rows], want, rtol=3e-2, atol=3e-2)
    _close(x.grad[:rows], xf.grad, rtol=3e-2, atol=3e-2)
    for got, ref_w in ((wg, wgf), (wu, wuf), (wd, wdf)):
        _close(got.grad, ref_w.grad, rtol=4e-2, atol=4e-2)


@pytest.mark.parametrize("experts", [8, 64])
def test_router_gate_projection_runs_on_the_native_gemm(native_lib, experts):
    """The router's gate is a GEMM with 8 .. 64 output columns: forward, input gradient and the (experts x dim)
    weight gradient go through the tcgen05 kernels and agree with fp32 matmuls."""
    from kempnerforge_b200.ops import functional as F

    torch.manual_seed(3)
    x = _rand(1000, 512).requires_grad_(True)
    w = _rand(experts, 512, scale=0.05).requires_grad_(True)
    before = native_lib.LAUNCH_COUNT
    y = F.linear(x, w)
    g = _rand(1000, experts)
    y.backward(g)
    assert native_lib.LAUNCH_COUNT >= before + 3 and native_lib.read_status() == 0
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    (xf @ wf.t()).backward(g.float())
    _close(y, xf @ wf.t())
    _close(x.grad, xf.grad)
    _close(w.grad, wf.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("counts", [[128, 128, 128, 128], [5, 0, 300, 77, 130, 1], [700, 24, 300]])
def test_grouped_swiglu_backward_epilogue_matches_two_kernel_path(native_lib, counts, b_mn):
    """Experts' down-projection input gradient with the SwiGLU gradient in its epilogue against the grouped GEMM
    followed by the ragged element-wise kernel (same roundings: bit-identical on the experts' rows)."""
    torch.manual_seed(2)
    e, d, f = len(counts), 192, 328 if not b_mn else 320
    rows = sum(counts)
    dy = _rand(rows + 40, d)
    wd = _rand(e, d, f, scale=0.1) if b_mn else _rand(e, f, d, scale=0.1)
    gu = _rand(rows + 40, 2 * f)
    off = torch.zeros(e + 1, dtype=torch.int32, device="cuda")
    off[1:] = torch.tensor(counts, device="cuda").cumsum(0)
    dh = native_lib.grouped_gemm(dy, wd, off, b_mn=b_mn)
    want = native_lib.swiglu_bwd_ragged(dh, gu, off)
    got = native_lib.grouped_swiglu_bwd(dy, wd, gu.clone(), off, b_mn=b_mn)
    assert native_lib.read_status() == 0
    assert torch.equal(got[:rows], want[:rows])
    assert torch.equal(got[rows:], gu[rows:])          # rows past the last expert are not touched


@pytest.mark.parametrize("shape", [(256, 256, 128), (512, 1536, 512), (1000, 768, 320)])
def test_gemm_swiglu_backward_epilogue_matches_two_kernel_path(native_lib, shape):
    """Input-gradient GEMM of the down projection with the SwiGLU gradient in its epilogue against the plain GEMM
    followed by the element-wise kernel (same roundings: bit-identical)."""
    m, f, k = shape
    dy, wd = _rand(m, k), _rand(k, f) * 0.1
    gu = _rand(m, 2 * f)
    want = native_lib.swiglu_bwd(native_lib.gemm(dy, wd, a_kmajor=True, b_kmajor=False, mode=2), gu.clone())
    got = native_lib.gemm_swiglu_bwd(dy, wd, gu.clone())
    assert native_lib.read_status() == 0
    assert torch.equal(got, want)


@pytest.mark.parametrize("shape,tall", [((256, 512), False), ((768, 320), False), ((1000, 1024), False),
                                        ((512, 256), True), ((2048, 520), True)])
def test_symmetric_product_matches_fp32_reference(native_lib, shape, tall):
    """alpha * X X^T + beta * R + diag * I (and the X^T X form) computed from the upper-triangle tiles only: against
    the fp32 product, exactly symmetric, and (without a polynomial) equal to the plain GEMM bit for bit."""
    x = _rand(*shape)
    n = shape[1] if tall else shape[0]
    xf = x.float()
    prod = xf.t() @ xf if tall else xf @ xf.t()
    got = native_lib.gemm_symm(x, tall)
    assert native_lib.read_status() == 0
    assert torch.equal(got, got.t())
    assert torch.allclose(got.float(), prod, rtol=8e-3, atol=0.05)   # bf16 rounding of an fp32 accumulation
    plain = native_lib.gemm(x, x, a_kmajor=False, b_kmajor=False, mode=2) if tall else native_lib.gemm(x, x, mode=2)
    assert torch.equal(torch.triu(got), torch.triu(plain))
    r = got
    poly = native_lib.gemm_symm(x, tall, residual=r, alpha=0.5, beta=-1.25, diag=3.0)
    want = 0.5 * prod - 1.25 * r.float() + 3.0 * torch.eye(n, device=x.device)
    assert torch.equal(poly, poly.t())
    assert torch.allclose(poly.float(), want, rtol=8e-3, atol=0.05)


def test_newton_schulz_on_symmetric_products_matches_fp32_iteration(native_lib):
    """The native Newton-Schulz iteration (symmetric Gram product, polynomial in the epilogue of the second product)
    against the plain fp32 formulation, wide and tall."""
    from kempnerforge_b200.ops import ref
    from kempnerforge_b200.training.optimizer import _newton_schulz_native

    for shape in ((512, 1536), (1024, 256)):
        g = torch.randn(*shape, device="cuda")
        got = _newton_schulz_native(g.to(torch.bfloat16), 5)
        assert got is not None and got.dtype == torch.bfloat16
        want = ref.newton_schulz(g.to(torch.bfloat16).float(), 5)
        err = (got.float() - want).norm() / want.norm()
        assert err < 5e-2, err
    assert native_lib.read_status() == 0


# --------------------------------------------------------------------------- vision-language models on one GPU
def _vlm_job(arch, **vlm_extra):
    from kempnerforge_b200.config import config_from_dict

    return config_from_dict({
        "model": dict(dim=256, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=512, ffn_hidden_dim=512, max_seq_len=128),
        "train": dict(batch_size=4, seq_len=64, max_steps=20, mixed_precision="bf16", seed=0),
        "optimizer": dict(lr=2e-3), "scheduler": dict(name="constant", warmup_steps=0),
        "vision_encoder": dict(type="random", feature_dim=64, num_tokens=16),
        "adapter": dict(type="mlp_2layer"),
        "vlm": dict(arch=arch, max_text_len=32, **vlm_extra),
        "metrics": dict(log_interval=1000),
    })


@pytest.mark.parametrize("arch", ["joint_decoder", "cross_attention", "mot", "moma"])
def test_vlm_architectures_build_and_train_on_the_gpu(native_lib, arch):
    """Every vision-language architecture is built on the device by the trainer (random encoder: no downloads),
    trains in bf16 and leaves the frozen encoder alone."""
    from kempnerforge_b200.training.trainer import Trainer

    extra = {"cross_attention_every_n_layers": 2} if arch == "cross_attention" else {}
    if arch == "moma":
        extra = {"moma_experts_per_modality": {"image": 2, "text": 2}, "moma_gumbel_noise": False}
    t = Trainer(_vlm_job(arch, freeze=[{"module": "vision_encoder", "frozen": True}], **extra), init_dist=False)
    assert all(p.is_cuda for p in t.model.parameters()) and t.model.vision_encoder.basis.is_cuda
    g = torch.Generator().manual_seed(0)
    batch = {"pixel_values": torch.rand(4, 3, 32, 32, generator=g), "input_ids": torch.randint(1, 512, (4, 32), generator=g)}
    batch["labels"] = batch["input_ids"].clone()
    losses = [t.train_step([batch])["loss"] for _ in range(10)]
    assert native_lib.read_status() == 0
    assert all(l == l for l in losses) and losses[-1] < losses[0] - 0.5, (arch, losses)


def test_vlm_all_padding_batch_is_harmless_on_the_gpu(native_lib):
    from kempnerforge_b200.training.trainer import Trainer

    t = Trainer(_vlm_job("joint_decoder"), init_dist=False)
    g = torch.Generator().manual_seed(1)
    px, ids = torch.rand(4, 3, 32, 32, generator=g), torch.randint(1, 512, (4, 32), generator=g)
    out = t.train_step([{"pixel_values": px, "input_ids": ids, "labels": torch.full((4, 32), -100)}])
    assert out["loss"] == 0.0 or out["loss"] == out["loss"]
    out = t.train_step([{"pixel_values": px, "input_ids": ids, "labels": ids.clone()}])
    assert out["loss"] == out["loss"] and out["loss"] > 0 and native_lib.read_status() == 0


# --------------------------------------------------------------------------- the rest of the user-facing paths on one GPU
def test_generation_evaluation_and_activation_capture_on_the_gpu(native_lib):
    """Decoding against per-layer KV caches, evaluation and activation capture run on the device through the same
    model object the trainer updates (bf16, native kernels where the shapes allow)."""
    from kempnerforge_b200.models.generate import generate
    from kempnerforge_b200.models.hooks import ActivationStore
    from kempnerforge_b200.training.eval import run_eval
    from kempnerforge_b200.training.loss import cross_entropy_loss
    from kempnerforge_b200.training.trainer import Trainer

    t = Trainer(_tiny_job(), init_dist=False)
    _overfit(t, steps=3)
    model = t.model
    prompt = torch.randint(0, 512, (2, 8), generator=torch.Generator().manual_seed(2)).cuda()
    out = generate(model, prompt, max_new_tokens=6, temperature=0.0)
    assert out.shape == (2, 14) and out.is_cuda and torch.equal(out[:, :8], prompt)
    assert int(out.min()) >= 0 and int(out.max()) < 512
    assert torch.equal(out, generate(model, prompt, max_new_tokens=6, temperature=0.0))       # greedy decoding repeats
    sampled = generate(model, prompt, max_new_tokens=4, temperature=0.8, top_k=20, top_p=0.9)
    assert sampled.shape == (2, 12)
    model.eval()
    with torch.no_grad():       # the first generated token is the argmax of a plain forward pass over the prompt
        last = model(prompt)[:, -1].float()
    chosen = last.gather(1, out[:, 8:9]).squeeze(1)     # (up to bf16 noise between the cached and the plain kernels)
    assert bool((last.max(-1).values - chosen <= 0.25).all()), (last.max(-1).values, chosen)
    g = torch.Generator().manual_seed(3)
    batches = []
    for _ in range(2):
        tok = torch.randint(0, 512, (4, 65), generator=g)
        batches.append({"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()})
    res = run_eval(model, batches, cross_entropy_loss, torch.device("cuda"), 3)
    assert res["eval/loss"] == res["eval/loss"] and res["eval/loss"] > 0
    assert abs(res["eval/perplexity"] - math.exp(res["eval/loss"])) <= 1e-3 * res["eval/perplexity"]
    store = ActivationStore(model, layers=["layers.0.attention", "layers.1.mlp", "norm"])
    store.enable()
    with torch.no_grad():
        model(prompt)
    store.disable()
    for name in ("layers.0.attention", "layers.1.mlp", "norm"):
        act = store.get(name)
        assert act is not None and tuple(act.shape) == (2, 8, 256), name
        assert bool(torch.isfinite(act.float()).all()), name
    assert native_lib.read_status() == 0


def test_checkpoint_round_trip_on_the_gpu_resumes_the_same_trajectory(native_lib, tmp_path):
    from kempnerforge_b200.training.trainer import Trainer

    def job():
        return _tiny_job(checkpoint=dict(dir=str(tmp_path / "ck"), interval=1000))

    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, 512, (4, 129), generator=g)
    batch = {"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}
    a = Trainer(job(), init_dist=False)
    a.setup_checkpointing()
    for _ in range(3):
        a.train_step([batch])
        a.step += 1
    a.save_checkpoint()
    a.ckpt.wait()
    want = [a.train_step([batch])["loss"] for _ in range(2)]
    b = Trainer(job(), init_dist=False)
    b.setup_checkpointing()
    assert b.step == 3
    got = [b.train_step([batch])["loss"] for _ in range(2)]
    assert native_lib.read_status() == 0
    for x, y in zip(got, want):
        assert abs(x - y) <= 2e-3 * max(1.0, abs(y)), (got, want)
