"""Mixture-of-experts feed-forward layer.

Dispatch is sort-based and ragged: the (token, slot) pairs are stably sorted by
expert, the rows are gathered once, the experts run as grouped GEMMs over
device-side segment offsets (no padding to the busiest expert, no host
synchronisation), and the result is un-permuted and reduced over the k slots in
a fixed order (deterministic — no atomics).

Parity: kempnerforge/model/moe.py:148-464 —
  capacity: cap = max(1, ceil(T*k/E*cf)); per (slot, expert) the first ``cap`` tokens in
    sequence order keep their weight, the rest get weight 0;
  optional per-expert gradient scale avg_tokens/count_e while training;
  packed experts ``up_w``/``gate_w`` (E, D, H), ``down_w`` (E, H, D); unpacked
    ``experts.{j}.{gate,up,down}_proj.weight``;
  ONE shared expert MLP (FQN ``shared_expert``) whatever ``moe_shared_experts`` says,
    optionally widened by that count (extension);
  expert-parallel attributes ``ep_world_size / ep_group / local_expert_start /
    num_local_experts``; ``aux_loss`` / ``z_loss`` / ``expert_counts`` forwarded from the router.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from kempnerforge_b200.models.mlp import SwiGLUMLP, build_mlp
from kempnerforge_b200.models.router import build_router
from kempnerforge_b200.ops import grouped


_HAS_GROUPED_MM = hasattr(torch, "_grouped_mm")   # the library's grouped GEMM (the fallback of the native kernels)


def _counts_tensor(tokens_per_expert, device) -> torch.Tensor:
    if torch.is_tensor(tokens_per_expert):
        return tokens_per_expert.to(device=device, dtype=torch.int64)
    return torch.tensor(list(tokens_per_expert), dtype=torch.int64, device=device)


def grouped_expert_forward(x_sorted: torch.Tensor, tokens_per_expert, experts) -> torch.Tensor:
    """Expert FFNs over rows sorted by expert, for a list of expert modules (``gate_proj``/``up_proj``/``down_proj``
    Linears, or ``up_proj``/``down_proj`` plus ``act``).  ``tokens_per_expert`` is a list or a device tensor of row
    counts in expert order.  Parity: kempnerforge/model/moe.py:20-83."""
    experts = list(experts.values()) if isinstance(experts, nn.ModuleDict) else list(experts)
    if x_sorted.shape[0] == 0:
        return torch.zeros_like(x_sorted)
    swiglu = hasattr(experts[0], "gate_proj")
    stack = lambda name: grouped.stack_expert_weights([getattr(e, name).weight for e in experts])  # noqa: E731
    return grouped.grouped_ffn(x_sorted, _counts_tensor(tokens_per_expert, x_sorted.device),
                               stack("gate_proj") if swiglu else None, stack("up_proj"), stack("down_proj"), "nk",
                               None if swiglu else experts[0].act)


def grouped_expert_forward_packed(x_sorted: torch.Tensor, tokens_per_expert, up_w: torch.Tensor, down_w: torch.Tensor,
                                  gate_w: torch.Tensor | None, activation) -> torch.Tensor:
    """Same over packed weights ``up_w``/``gate_w`` (E, dim, hidden) and ``down_w`` (E, hidden, dim); ``activation``
    is used when ``gate_w`` is None.  Parity: kempnerforge/model/moe.py:86-145."""
    if x_sorted.shape[0] == 0:
        return torch.zeros_like(x_sorted)
    return grouped.grouped_ffn(x_sorted, _counts_tensor(tokens_per_expert, x_sorted.device), gate_w, up_w, down_w, "kn",
                               None if gate_w is not None else activation)


def apply_capacity(weights: torch.Tensor, indices: torch.Tensor, num_experts: int, capacity_factor: float):
    """Zero the routing weight of tokens beyond each expert's per-slot capacity (device only)."""
    t, k = indices.shape
    cap = max(1, math.ceil(t * k / num_experts * capacity_factor))
    if indices.is_cuda and indices.dtype == torch.int64:
        from kempnerforge_b200.ops import cuda as kc
        from kempnerforge_b200.ops import functional as _F

        if kc.available() and not _F._FORCE_REF and getattr(kc.lib(), "kf_moe_capacity_mask", None) is not None:
            keep = kc.moe_capacity_mask(indices.contiguous(), num_experts, cap)   # one kernel, no (T, k, E) one-hot
            return weights * keep.to(weights.dtype), indices
    onehot = torch.nn.functional.one_hot(indices, num_experts)  # (T, k, E)
    rank = (onehot.cumsum(dim=0) * onehot).sum(dim=-1) - 1  # arrival order within (slot, expert)
    keep = rank < cap
    return weights * keep.to(weights.dtype), indices


_apply_capacity = apply_capacity


class MoEMLP(nn.Module):
    def __init__(
        self,
        router: nn.Module,
        experts: nn.ModuleList,
        shared_expert: nn.Module | None = None,
        capacity_factor: float = 0.0,
        gradient_scale: bool = False,
        packed_experts: bool = False,
    ) -> None:
        super().__init__()
        self.router = router
        self.shared_expert = shared_expert
        self.num_experts = len(experts)
        self.capacity_factor = capacity_factor
        self.gradient_scale = gradient_scale
        self.packed_experts = packed_experts
        self.ep_world_size = 1
        self.ep_group = None
        self.ep_comm = None  # device-side dispatch context (set by apply_expert_parallel)
        self.local_expert_start = 0
        self.num_local_experts = len(experts)
        self.tp_input = None  # TPContext of a tensor-parallel model (experts themselves are replicated)
        self._is_swiglu = isinstance(experts[0], SwiGLUMLP) or hasattr(experts[0], "gate_proj")
        if packed_experts:
            stack = lambda name: nn.Parameter(  # noqa: E731
                torch.stack([getattr(e, name).weight.detach().t().contiguous() for e in experts])
            )
            self.up_w = stack("up_proj")
            self.down_w = stack("down_proj")
            if self._is_swiglu:
                self.gate_w = stack("gate_proj")
            else:
                self._packed_activation = experts[0].act
        else:
            self.experts = experts

    # -- expert weights in grouped-GEMM form ------------------------------------------
    def expert_weights(self):
        """(gate, up, down, layout): layout 'kn' = (E, in, out) packed, 'nk' = (E, out, in) stacked Linears."""
        if self.packed_experts:
            return (self.gate_w if self._is_swiglu else None), self.up_w, self.down_w, "kn"
        stack = lambda name: grouped.stack_expert_weights([getattr(e, name).weight for e in self.expert_modules()])  # noqa: E731
        gate = stack("gate_proj") if self._is_swiglu else None
        return gate, stack("up_proj"), stack("down_proj"), "nk"

    def _activation(self):
        if self._is_swiglu:
            return None
        return self._packed_activation if self.packed_experts else self.expert_modules()[0].act

    def expert_modules(self) -> list[nn.Module]:
        """Local expert modules in expert order (a ModuleList, or a ModuleDict keyed by global index under EP)."""
        ex = self.experts
        return list(ex.values()) if isinstance(ex, nn.ModuleDict) else list(ex)

    def run_experts(self, x_sorted: torch.Tensor, counts: torch.Tensor, offsets: torch.Tensor | None = None) -> torch.Tensor:
        """Grouped expert FFN over rows already sorted by (local) expert.  ``offsets`` (int32 (E + 1), device): the
        row ranges when they are already known; ``x_sorted`` may then be longer than ``offsets[-1]``."""
        gate, up, down, layout = self.expert_weights()
        return grouped.grouped_ffn(x_sorted, counts, gate, up, down, layout, self._activation(), offsets=offsets)

    def _local_forward(self, x_flat, weights, indices):
        t, k = indices.shape
        from kempnerforge_b200.ops import moe_ops

        if (moe_ops.native_ok(x_flat, self.num_experts, k) and x_flat.dtype == torch.bfloat16
                and x_flat.shape[1] % 8 == 0 and not (self.gradient_scale and self.training)):
            # device-side stable sort by expert, row gather, grouped expert GEMMs, weighted combine
            offsets, row_of_slot, slot_of_row = moe_ops.sort_by_expert(indices, self.num_experts)
            counts = (offsets[1:] - offsets[:-1]).to(torch.int64)
            x_sorted = moe_ops.gather_rows(x_flat, slot_of_row, row_of_slot, k)
            y = self.run_experts(x_sorted, counts, offsets=offsets)
            return moe_ops.combine_rows(y, weights, row_of_slot, slot_of_row)
        flat_e = indices.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        token_of_row = order // k
        counts = torch.bincount(flat_e, minlength=self.num_experts)
        y = self.run_experts(x_flat.index_select(0, token_of_row), counts)
        if self.gradient_scale and self.training:
            avg = (t * k) / max(1, self.num_experts)
            scale = avg / counts.clamp(min=1).to(y.dtype)
            y = y * scale[flat_e[order]].unsqueeze(-1)
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(order.numel(), device=order.device)
        y = y.index_select(0, inverse).view(t, k, -1)
        return (y * weights.unsqueeze(-1).to(y.dtype)).sum(dim=1)

    @property
    def aux_loss(self) -> torch.Tensor:
        return self.router.aux_loss

    @property
    def z_loss(self) -> torch.Tensor:
        return self.router.z_loss

    @property
    def expert_counts(self) -> torch.Tensor:
        return self.router.expert_counts

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, s, d = x.shape
        x_flat = x.reshape(b * s, d)
        weights, indices = self.router(x_flat)
        if self.capacity_factor > 0:
            weights, indices = apply_capacity(weights, indices, self.num_experts, self.capacity_factor)
        if self.ep_world_size > 1:
            from kempnerforge_b200.parallel.expert_parallel import ep_dispatch_and_compute

            out = ep_dispatch_and_compute(x_flat, weights, indices, self)
        else:
            out = self._local_forward(x_flat, weights, indices)
        if self.shared_expert is not None:
            out = out + self.shared_expert(x_flat)
        return out.view(b, s, d)


def build_moe(
    dim: int,
    hidden_dim: int,
    num_experts: int,
    top_k: int,
    activation: str = "silu",
    router_type: str = "softmax_topk",
    shared_experts: int = 0,
    capacity_factor: float = 0.0,
    gradient_scale: bool = False,
    sequence_aux_loss_weight: float = 0.0,
    bias_schedule: str = "constant",
    packed_experts: bool = False,
    shared_expert_widen: bool = False,
) -> MoEMLP:
    kwargs = {}
    if router_type == "sigmoid_topk":
        kwargs = {"sequence_aux_loss_weight": sequence_aux_loss_weight, "bias_schedule": bias_schedule}
    router = build_router(router_type, dim, num_experts, top_k, **kwargs)
    experts = nn.ModuleList(build_mlp(dim, hidden_dim, activation) for _ in range(num_experts))
    shared = None
    if shared_experts > 0:
        width = hidden_dim * shared_experts if shared_expert_widen else hidden_dim
        shared = build_mlp(dim, width, activation)
    return MoEMLP(router, experts, shared, capacity_factor, gradient_scale, packed_experts)
