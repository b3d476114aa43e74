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
    dist.all_reduce(x, group=group)  # gloo has no reduce-scatter; NCCL paths are replaced by fused kernels
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

    def before_column_parallel(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            return _GatherSeq.apply(x, 1, self.group)
        return _AllReduceBwd.apply(x, self.group)

    def after_row_parallel(self, y: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            return _ScatterSumSeq.apply(y, 1, self.group)
        return _AllReduceFwd.apply(y, self.group)

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


def get_tp_mesh(mesh):
    if mesh is None or "tp" not in (mesh.mesh_dim_names or ()):
        return None
    return mesh["tp"]


def apply_tensor_parallel(model: nn.Module, mesh, sequence_parallel: bool | None = None) -> TPContext | None:
    group, size, _ = mesh_dim(mesh, "tp")
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
        if getattr(p, "_kf_tp_partial_grad", False):
            g = getattr(p, "_kf_grad", None) if getattr(p, "_kf_grad_live", False) else p.grad
            if g is not None:
                dist.all_reduce(g, group=ctx.group)


# --------------------------------------------------------------------------- vocabulary-parallel loss
class _VocabParallelCE(torch.autograd.Function):
    """Cross entropy over logits whose vocabulary dimension is sharded: ranks exchange only the per-token
    maximum, sum of exponentials and picked logit instead of gathering (tokens, vocab) logits."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_start, group, z_weight):
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
        probs, local_label, mine, valid, lse, n = ctx.saved_tensors
        grad = probs * (1.0 + 2.0 * ctx.z_weight * lse)[:, None]
        rows = torch.nonzero(mine, as_tuple=False).squeeze(-1)
        grad[rows, local_label[rows]] -= 1.0
        grad = grad * (valid.float() / n)[:, None] * g
        return grad.to(probs.dtype), None, None, None, None


def vocab_parallel_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ctx: TPContext, z_loss_weight: float = 0.0):
    """logits (tokens, vocab / tp) of this rank, labels (tokens,) with global ids."""
    v_local = logits.shape[-1]
    out = _VocabParallelCE.apply(logits, labels, ctx.rank * v_local, ctx.group, float(z_loss_weight))
    return out
