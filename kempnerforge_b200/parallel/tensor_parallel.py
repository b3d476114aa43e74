"""Megatron-style tensor parallelism with optional sequence parallelism.

Column-parallel weights (q/k/v, gate/up, vocabulary rows of the head) keep a slice of their output
features; row-parallel weights (o, down) keep a slice of their input features.  With sequence
parallelism the activations between blocks are sharded along the sequence: a column-parallel GEMM
is preceded by an all-gather of the sequence shards, a row-parallel GEMM is followed by a
reduce-scatter, and the norms run on S/tp tokens.  Without it the input is replicated and the
row-parallel output is all-reduced.

The collectives are autograd functions over ``torch.distributed`` (NCCL on GPUs, gloo on CPU); the
fused all-gather->GEMM / GEMM->reduce-scatter kernels plug in behind the same ``TPContext`` calls.

Parameters that see only a part of the tokens (norm weights under sequence parallelism) or that are
replicated but receive partial gradients are tagged ``_kf_tp_partial_grad``; ``sync_partial_grads``
sums those gradients over the TP group after backward.  Sharded parameters carry
``_kf_shard = (mesh_dim_name, tensor_dim)`` so checkpoints can describe them as sharded tensors.

Parity: kempnerforge/distributed/tensor_parallel.py:52-178 (same plan: q/k/v/gate/up column-wise,
o/down row-wise, MoE blocks: attention only, sequence parallelism off for pipeline stages, tied
embeddings and MoE models, vocabulary-parallel output head).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch import nn

from kempnerforge_b200.parallel.setup import mesh_dim


# --------------------------------------------------------------------------- collectives with gradients
def _all_gather_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    x = x.contiguous()
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=dim)


def _reduce_scatter_dim(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    if x.is_cuda and "nccl" in str(dist.get_backend(group)):
        parts = [p.contiguous() for p in x.chunk(world, dim=dim)]
        out = torch.empty_like(parts[rank])
        dist.reduce_scatter(out, parts, group=group)
        return out
    dist.all_reduce(x, group=group)  # gloo has no reduce-scatter
    return x.chunk(world, dim=dim)[rank].contiguous()


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _all_gather_dim(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim(g.clone(), ctx.dim, ctx.group), None, None


class _GatherReplicated(torch.autograd.Function):
    """All-gather whose result is consumed identically on every rank: backward keeps the local chunk."""

    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _all_gather_dim(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        world, rank = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        return g.chunk(world, dim=ctx.dim)[rank].contiguous(), None, None


class _ScatterSumSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _reduce_scatter_dim(x.clone(), dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.dim, ctx.group), None, None


class _AllReduceFwd(torch.autograd.Function):
    """Sum in forward, identity in backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _AllReduceBwd(torch.autograd.Function):
    """Identity in forward, sum in backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _SliceSeq(torch.autograd.Function):
    """Keep this rank's sequence chunk of a replicated tensor; backward gathers the chunks."""

    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        return x.chunk(world, dim=dim)[rank].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.dim, ctx.group), None, None


class TPContext:
    """What a sharded layer needs to know: the group, its size and whether activations are sequence-sharded."""

    def __init__(self, group, sequence_parallel: bool) -> None:
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.sequence_parallel = sequence_parallel
        self._fused: bool | None = None      # decided at the first call (needs a tensor to look at)
        self._ctx: dict[str, object] = {}    # symmetric-memory buffers of the fused kernels

    def before_column_parallel(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            return _GatherSeq.apply(x, 1, self.group)
        return _AllReduceBwd.apply(x, self.group)

    def after_row_parallel(self, y: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            return _ScatterSumSeq.apply(y, 1, self.group)
        return _AllReduceFwd.apply(y, self.group)

    # ---- fused GEMM + collective kernels (sequence parallelism on GPUs of one NVLink domain) -------------
    def _fused_ok(self, x: torch.Tensor, seq_shard: int, k: int) -> bool:
        if self._fused is None:
            self._fused = (os.environ.get("KF_TP_FUSED", "1") != "0" and self.sequence_parallel and x.is_cuda
                           and "nccl" in str(dist.get_backend(self.group))
                           and int(os.environ.get("LOCAL_WORLD_SIZE", "0") or 0) == int(os.environ.get("WORLD_SIZE", "1")))
        return bool(self._fused) and x.dtype == torch.bfloat16 and seq_shard % 128 == 0 and k % 32 == 0

    def _context(self, kind: str, tokens: int, dim: int, device):
        from kempnerforge_b200.comm.fused_tp import AgGemmContext, GemmRSContext

        cur = self._ctx.get(kind)
        if cur is None or tokens > cur.max_tokens or dim > cur.max_dim:
            cls = AgGemmContext if kind == "ag" else GemmRSContext
            if cur is not None:
                tokens, dim = max(tokens, cur.max_tokens), max(dim, cur.max_dim)
            cur = self._ctx[kind] = cls(self.group, device, tokens, dim)
        return cur

    def column_linear(self, x: torch.Tensor, weights: list[torch.Tensor]) -> torch.Tensor:
        """Column-parallel Linear on a sequence-sharded (B, S/tp, K) input: one kernel gathers and multiplies when
        the fused path applies, otherwise all-gather followed by the GEMM."""
        from kempnerforge_b200.ops import functional as F

        if x.dim() == 3 and self._fused_ok(x, x.shape[1], x.shape[2]) and all(w.dtype == torch.bfloat16 for w in weights):
            return _FusedColumnLinearFn.apply(x, self, *weights)
        return F.fused_linear(self.before_column_parallel(x), weights)

    def row_linear(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """Row-parallel Linear whose (B, S, D) partial sums are reduce-scattered along the sequence."""
        from kempnerforge_b200.ops import functional as F

        if (x.dim() == 3 and x.shape[1] % self.size == 0 and self._fused_ok(x, x.shape[1] // self.size, 32)
                and weight.dtype == torch.bfloat16 and x.shape[2] % 8 == 0 and weight.shape[0] % 8 == 0):
            return _FusedRowLinearFn.apply(x, self, weight)
        return self.after_row_parallel(F.linear(x, weight))

    def scatter_sequence(self, x: torch.Tensor) -> torch.Tensor:
        return _SliceSeq.apply(x, 1, self.group) if self.sequence_parallel else x

    def gather_sequence(self, x: torch.Tensor) -> torch.Tensor:
        return _GatherSeq.apply(x, 1, self.group) if self.sequence_parallel else x

    def head_input(self, h: torch.Tensor) -> torch.Tensor:
        """Hidden states entering the vocabulary-parallel head.  Under sequence parallelism the preceding
        sequence gather already sums the per-shard gradients; otherwise they are summed here."""
        return h if self.sequence_parallel else _AllReduceBwd.apply(h, self.group)

    def gather_vocab(self, logits: torch.Tensor) -> torch.Tensor:
        return _GatherReplicated.apply(logits, logits.dim() - 1, self.group)


class _FusedColumnLinearFn(torch.autograd.Function):
    """y = gather_seq(x) @ [W_0; W_1; ...]ᵀ with the gather inside the GEMM kernel.  Backward: the input gradient is a
    GEMM whose epilogue reduce-scatters (``kf_gemm_rs``); the weight gradient all-gathers the input with the library."""

    @staticmethod
    def forward(ctx, x, tp, *weights):
        from kempnerforge_b200.ops import cuda as kc
        from kempnerforge_b200.ops import functional as F

        b, s_local, k = x.shape
        w = F._stack_weight_rows(weights)
        x2 = x.reshape(b * s_local, k)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        t = b * s_local * tp.size
        y = kc.all_gather_gemm(x2, w, tp._context("ag", t, k, x.device), s_local * tp.size)
        ctx.save_for_backward(x2, *weights)
        ctx.tp, ctx.dims = tp, (b, s_local, k)
        # rows come out in (b, s) order of the full sequence
        return y.view(b, s_local * tp.size, w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from kempnerforge_b200.ops import cuda as kc
        from kempnerforge_b200.ops import functional as F

        x2, *weights = ctx.saved_tensors
        tp, (b, s_local, k) = ctx.tp, ctx.dims
        w = F._stack_weight_rows(weights)
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            n_local = w.shape[0]
            if n_local % 64 == 0 and k % 8 == 0:
                # dx_partial = dy @ W reduced over the ranks and scattered along the sequence inside the GEMM
                dx = kc.gemm_reduce_scatter(dy2, w, tp._context("rs", dy2.shape[0], k, dy2.device), s_local * tp.size,
                                            w_kn=True).view(b, s_local, k)
            else:
                dx_full = kc.gemm(dy2, w, a_kmajor=True, b_kmajor=False).view(b, s_local * tp.size, k)
                dx = _reduce_scatter_dim(dx_full, 1, tp.group)
        wgrads = [None] * len(weights)
        if any(ctx.needs_input_grad[2:]):
            x_full = _all_gather_dim(x2.view(b, s_local, k), 1, tp.group).reshape(-1, k)
            wgrads = F._linear_weight_grads(kc, dy2, x_full, weights, ctx.needs_input_grad[2:])
        return (dx, None, *wgrads)


class _FusedRowLinearFn(torch.autograd.Function):
    """out = reduce_scatter_seq(x @ Wᵀ) with the tiles pushed to their owners from the GEMM epilogue.  Backward: the
    input gradient gathers the output gradient inside its GEMM (``kf_ag_gemm``); the weight gradient uses a library
    all-gather and a plain GEMM."""

    @staticmethod
    def forward(ctx, x, tp, weight):
        from kempnerforge_b200.ops import cuda as kc

        b, s, k = x.shape
        x2 = x.reshape(b * s, k)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        d = weight.shape[0]
        out = kc.gemm_reduce_scatter(x2, weight, tp._context("rs", b * s, d, x.device), s)
        ctx.save_for_backward(x2, weight)
        ctx.tp, ctx.dims = tp, (b, s, k, d)
        return out.view(b, s // tp.size, d)

    @staticmethod
    def backward(ctx, dy):
        from kempnerforge_b200.ops import cuda as kc
        from kempnerforge_b200.ops import functional as F

        x2, weight = ctx.saved_tensors
        tp, (b, s, k, d) = ctx.tp, ctx.dims
        dx = None
        dy_full = None
        if ctx.needs_input_grad[0]:
            if d % 64 == 0 and k % 8 == 0:
                # dx = gather_seq(dy) @ W with the gather inside the GEMM (W read with its input dim contiguous)
                dy2 = dy.reshape(-1, d)
                if not dy2.is_contiguous():
                    dy2 = dy2.contiguous()
                dx = kc.all_gather_gemm(dy2, weight, tp._context("ag", b * s, d, dy.device), s, w_kn=True).view(b, s, k)
            else:
                dy_full = _all_gather_dim(dy, 1, tp.group).reshape(b * s, d)
                dx = kc.gemm(dy_full, weight, a_kmajor=True, b_kmajor=False).view(b, s, k)
        gw = None
        if ctx.needs_input_grad[2]:
            if dy_full is None:
                dy_full = _all_gather_dim(dy, 1, tp.group).reshape(b * s, d)
            (gw,) = F._linear_weight_grads(kc, dy_full, x2, [weight], [True])
        return dx, None, gw


# --------------------------------------------------------------------------- sharding the weights
def _shard_param(module: nn.Module, name: str, dim: int, ctx: TPContext) -> None:
    p = getattr(module, name)
    if p.shape[dim] % ctx.size:
        raise ValueError(f"cannot shard {tuple(p.shape)} along dim {dim} over tp={ctx.size}")
    local = p.detach().chunk(ctx.size, dim=dim)[ctx.rank].clone()
    new = nn.Parameter(local, requires_grad=p.requires_grad)
    new._kf_shard = ("tp", dim)
    new._kf_global_shape = tuple(p.shape)
    setattr(module, name, new)


def build_block_tp_plan(block: nn.Module) -> dict[str, str]:
    """{sub-module path: "colwise" | "rowwise"} for one transformer block (MoE blocks: attention only)."""
    plan = {f"attention.{n}_proj": "colwise" for n in ("q", "k", "v")}
    plan["attention.o_proj"] = "rowwise"
    mlp = getattr(block, "mlp", None)
    if mlp is not None and hasattr(mlp, "down_proj") and not hasattr(mlp, "router"):
        if hasattr(mlp, "gate_proj"):
            plan["mlp.gate_proj"] = "colwise"
        plan["mlp.up_proj"] = "colwise"
        plan["mlp.down_proj"] = "rowwise"
    return plan


_build_block_tp_plan = build_block_tp_plan


def get_tp_mesh(device_mesh):
    if device_mesh is None or "tp" not in (device_mesh.mesh_dim_names or ()):
        return None
    return device_mesh["tp"]


def apply_tensor_parallel(model: nn.Module, device_mesh, sequence_parallel: bool | None = None) -> TPContext | None:
    group, size, _ = mesh_dim(device_mesh, "tp")
    if size <= 1:
        return None
    cfg = getattr(model, "config", None)
    is_moe = bool(cfg is not None and cfg.is_moe)
    tied = bool(cfg is not None and cfg.tie_embeddings)
    is_pp_stage = getattr(model, "is_pipeline_stage", False)
    if sequence_parallel is None:
        sequence_parallel = not (is_moe or tied or is_pp_stage)
    ctx = TPContext(group, sequence_parallel)
    for block in model.layers.values():
        for path, kind in build_block_tp_plan(block).items():
            owner = block.get_submodule(path)
            _shard_param(owner, "weight", 0 if kind == "colwise" else 1, ctx)
        block.attention.tp = ctx
        if "mlp.down_proj" in build_block_tp_plan(block):
            block.mlp.tp = ctx
        else:
            block.mlp.tp_input = ctx  # experts stay replicated across TP ranks; only the activations move
        if sequence_parallel:
            for norm in (block.attention_norm, block.mlp_norm):
                for p in norm.parameters():
                    p._kf_tp_partial_grad = True
    if sequence_parallel and getattr(model, "norm", None) is not None:
        for p in model.norm.parameters():
            p._kf_tp_partial_grad = True
    if getattr(model, "output_head", None) is not None and not tied:
        _shard_param(model.output_head.proj, "weight", 0, ctx)  # vocabulary-parallel head
        model.output_head.tp = ctx
    model.tp = ctx
    return ctx


def sync_partial_grads(model: nn.Module) -> None:
    """Sum, over the TP group, the gradients of parameters that only saw part of the tokens."""
    ctx = getattr(model, "tp", None)
    if ctx is None:
        return
    for p in model.parameters():
        if getattr(p, "_kf_tp_partial_grad", False) and not getattr(p, "_kf_tp_synced", False):
            g = getattr(p, "_kf_grad", None) if getattr(p, "_kf_grad_live", False) else p.grad
            if g is not None:
                dist.all_reduce(g, group=ctx.group)


def sync_partial_grads_of(params, ctx) -> None:
    """The same for one block's parameters, as soon as its backward has finished (so that the block's data-parallel
    reduction can start while the rest of the backward runs); marks them so the end-of-backward pass skips them."""
    for p in params:
        if getattr(p, "_kf_tp_partial_grad", False) and not getattr(p, "_kf_tp_synced", False):
            g = getattr(p, "_kf_grad", None) if getattr(p, "_kf_grad_live", False) else p.grad
            if g is not None:
                dist.all_reduce(g, group=ctx.group)
                p._kf_tp_synced = True


# --------------------------------------------------------------------------- vocabulary-parallel loss
class _VocabParallelCE(torch.autograd.Function):
    """Cross entropy over logits whose vocabulary dimension is sharded: ranks exchange only the per-token
    maximum, sum of exponentials and picked logit instead of gathering (tokens, vocab) logits."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group, z_weight):
        ctx.native = False
        if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(-1) == 1 and logits.stride(0) % 8 == 0:
            from kempnerforge_b200.ops import cuda as kc
            from kempnerforge_b200.ops import functional as _F

            if kc.available() and not _F._FORCE_REF and getattr(kc.lib(), "kf_ce_vp_stats_bf16", None) is not None:
                # kernels: per-row (max, sum exp, picked) of the local shard; two (T,) all-reduces; gradient in place
                labels = labels.contiguous()
                row_max, row_sum, picked = kc.ce_vp_stats(logits, labels, vocab_start)
                gmax = row_max.clone()
                dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
                both = torch.stack([row_sum * torch.exp(row_max - gmax), picked])
                dist.all_reduce(both, group=group)
                lse = gmax + torch.log(both[0])
                valid = labels != -100
                n = valid.sum().clamp_min(1).float()
                zero = torch.zeros_like(lse)
                nll = torch.where(valid, lse - both[1], zero).sum() / n
                z = torch.where(valid, lse * lse, zero).sum() / n
                ctx.native, ctx.z_weight, ctx.vocab_start = True, z_weight, vocab_start
                ctx.save_for_backward(logits, labels, lse, (1.0 / n).reshape(1))
                return nll + z_weight * z
        lf = logits.float()
        local_max = lf.max(dim=-1).values
        gmax = local_max.clone()
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
        ex = torch.exp(lf - gmax[:, None])
        sumexp = ex.sum(dim=-1)
        dist.all_reduce(sumexp, group=group)
        lse = gmax + torch.log(sumexp)
        v_local = lf.shape[-1]
        local_label = labels - vocab_start
        mine = (local_label >= 0) & (local_label < v_local)
        picked = torch.where(mine, lf.gather(-1, local_label.clamp(0, v_local - 1)[:, None]).squeeze(-1), torch.zeros_like(lse))
        dist.all_reduce(picked, group=group)
        valid = labels != -100
        n = valid.sum().clamp_min(1).float()
        nll = torch.where(valid, lse - picked, torch.zeros_like(lse)).sum() / n
        z = torch.where(valid, lse * lse, torch.zeros_like(lse)).sum() / n
        ctx.save_for_backward(ex / sumexp[:, None], local_label, mine, valid, lse, n)
        ctx.z_weight = z_weight
        return nll + z_weight * z

    @staticmethod
    def backward(ctx, g):
        if ctx.native:
            from kempnerforge_b200.ops import cuda as kc

            logits, labels, lse, inv_n = ctx.saved_tensors
            # the logits feed nothing but this loss: their storage becomes the gradient
            grad = kc.ce_vp_bwd(logits, labels, ctx.vocab_start, lse, inv_n, g.reshape(1).float().contiguous(), ctx.z_weight)
            return grad, None, None, None, None
        probs, local_label, mine, valid, lse, n = ctx.saved_tensors
        grad = probs * (1.0 + 2.0 * ctx.z_weight * lse)[:, None]
        # subtract the one-hot without a data-dependent shape (no host read): rows whose label lives elsewhere add 0
        grad.scatter_add_(1, local_label.clamp(0, grad.shape[1] - 1)[:, None], -mine.to(grad.dtype)[:, None])
        grad = grad * (valid.float() / n)[:, None] * g
        return grad.to(probs.dtype), None, None, None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ctx: TPContext, z_loss_weight: float = 0.0):
    """logits (tokens, vocab / tp) of this rank, labels (tokens,) with global ids."""
    v_local = logits.shape[-1]
    out = _VocabParallelCE.apply(logits, labels, ctx.rank * v_local, ctx.group, float(z_loss_weight))
    return out
