"""Top-k routers for mixture-of-experts layers.

Both routers return ``(weights, indices)`` of shape (tokens, top_k) and leave
``aux_loss``, ``z_loss`` and ``expert_counts`` on the module for the training
loop.  Everything stays on the device: counts come from ``bincount`` rather
than a (tokens, k, experts) one-hot, and nothing is read back to the host.

Parity: kempnerforge/model/router.py:15-214 —
  softmax router: softmax -> top-k -> renormalise; Switch aux loss E*sum(f_i*P_i);
  sigmoid router (DeepSeek-V3): sigmoid(logits + expert_bias) -> top-k -> renormalise,
  EMA of utilisation nudges ``expert_bias`` (a Parameter) in place under no_grad,
  bias-rate schedules constant / cosine_decay / linear_warmup, optional sequence aux loss;
  both: z-loss mean(logsumexp(logits)^2).
"""

from __future__ import annotations

import math

import torch
from torch import nn

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.ops import functional as F


def _counts(indices: torch.Tensor, num_experts: int) -> torch.Tensor:
    return torch.bincount(indices.reshape(-1), minlength=num_experts).float()


class SoftmaxTopKRouter(nn.Module):
    def __init__(self, dim: int, num_experts: int, top_k: int) -> None:
        super().__init__()
        self.gate = nn.Linear(dim, num_experts, bias=False)
        self.num_experts = num_experts
        self.top_k = top_k
        self.aux_loss = torch.tensor(0.0)
        self.z_loss = torch.tensor(0.0)
        self.expert_counts = torch.zeros(num_experts)

    def forward(self, x: torch.Tensor):
        logits = F.linear(x, self.gate.weight)   # the native GEMM on a GPU (the gate has no bias)
        from kempnerforge_b200.ops import moe_ops

        if moe_ops.native_ok(logits, self.num_experts, self.top_k):
            # one kernel: softmax, top-k, renormalised weights, counts, mean probabilities, z-loss
            weights, indices, counts, pmean, z = moe_ops.route(logits, None, False, self.top_k)
            self.expert_counts = counts.detach()
            frac = counts / (x.shape[0] * self.top_k)
            self.aux_loss = self.num_experts * (frac.detach() * pmean).sum()
            self.z_loss = z
            return weights.to(x.dtype), indices
        probs = torch.softmax(logits.float(), dim=-1)
        weights, indices = torch.topk(probs, self.top_k, dim=-1)
        weights = (weights / weights.sum(dim=-1, keepdim=True)).to(x.dtype)
        counts = _counts(indices, self.num_experts)
        self.expert_counts = counts.detach()
        frac = counts / (x.shape[0] * self.top_k)
        self.aux_loss = self.num_experts * (frac.detach() * probs.mean(dim=0)).sum()
        self.z_loss = torch.logsumexp(logits.float(), dim=-1).pow(2).mean()
        return weights, indices


class SigmoidTopKRouter(nn.Module):
    def __init__(
        self,
        dim: int,
        num_experts: int,
        top_k: int,
        bias_update_rate: float = 0.001,
        ema_decay: float = 0.99,
        sequence_aux_loss_weight: float = 0.0,
        bias_schedule: str = "constant",
    ) -> None:
        super().__init__()
        self.gate = nn.Linear(dim, num_experts, bias=False)
        self.num_experts = num_experts
        self.top_k = top_k
        self.bias_update_rate = bias_update_rate
        self.ema_decay = ema_decay
        self.sequence_aux_loss_weight = sequence_aux_loss_weight
        self.bias_schedule = bias_schedule
        self._step = 0
        self._max_steps = 1
        self._bias_fifo: list[torch.Tensor] = []  # biases used by checkpointed forward passes awaiting recomputation
        self.expert_bias = nn.Parameter(torch.zeros(num_experts))
        self.register_buffer("expert_ema", torch.full((num_experts,), 1.0 / num_experts))
        self.aux_loss = torch.tensor(0.0)
        self.z_loss = torch.tensor(0.0)
        self.expert_counts = torch.zeros(num_experts)

    def set_step(self, step: int, max_steps: int) -> None:
        self._step = step
        self._max_steps = max(1, max_steps)
        self._bias_fifo.clear()  # every backward of the previous step has run

    def _effective_bias_rate(self) -> float:
        t = self._step / self._max_steps
        shape = {
            "constant": 1.0,
            "cosine_decay": 0.5 * (1.0 + math.cos(math.pi * t)),
            "linear_warmup": min(1.0, 10.0 * t),
        }.get(self.bias_schedule, 1.0)
        return self.bias_update_rate * shape

    def _bias_for_this_pass(self) -> tuple[torch.Tensor, bool]:
        """The balancing bias this pass routes with, and whether this pass may update the router's state.

        Inside an activation-checkpointed block the forward runs twice.  The first pass records the bias it
        used (it nudges the parameter right afterwards); the recomputation routes with that recorded value, so
        both passes pick the same experts, and leaves the moving average and the bias alone.  First-in first-out
        matches every schedule in which backward passes run in the order of their forward passes (plain
        accumulation, GPipe, 1F1B)."""
        from kempnerforge_b200.models import recompute

        ph = recompute.phase()
        if ph == "forward" and self.training:
            self._bias_fifo.append(self.expert_bias.detach().clone())
            return self.expert_bias, True
        if ph == "recompute" and self._bias_fifo:
            used = self._bias_fifo.pop(0)
            # same value as in the first pass, gradient still reaches the parameter
            return self.expert_bias + (used - self.expert_bias).detach(), False
        return self.expert_bias, ph != "recompute"

    def forward(self, x: torch.Tensor):
        logits = F.linear(x, self.gate.weight)   # the native GEMM on a GPU (the gate has no bias)
        from kempnerforge_b200.ops import moe_ops

        bias, may_update = self._bias_for_this_pass()
        native = moe_ops.native_ok(logits, self.num_experts, self.top_k)
        if native:
            weights, indices, counts, smean, z = moe_ops.route(logits, bias, True, self.top_k)
            weights = weights.to(x.dtype)
        else:
            scores = torch.sigmoid(logits.float() + bias.float())
            weights, indices = torch.topk(scores, self.top_k, dim=-1)
            weights = (weights / weights.sum(dim=-1, keepdim=True)).to(x.dtype)
            counts = _counts(indices, self.num_experts)
            smean = None
        self.expert_counts = counts.detach()
        util = counts / (x.shape[0] * self.top_k + 1e-8)
        if self.training and may_update:
            with torch.no_grad():
                self.expert_ema.lerp_(util.to(self.expert_ema.dtype), 1.0 - self.ema_decay)
                nudge = self._effective_bias_rate() * (1.0 / self.num_experts - self.expert_ema.float())
                self.expert_bias.add_(nudge.to(self.expert_bias.dtype))
        if self.sequence_aux_loss_weight > 0:
            mean_scores = smean if native else scores.mean(dim=0)
            balance = self.num_experts * (util.detach() * mean_scores).sum()
            self.aux_loss = self.sequence_aux_loss_weight * balance
        else:
            self.aux_loss = torch.zeros((), device=x.device)
        self.z_loss = z if native else torch.logsumexp(logits.float(), dim=-1).pow(2).mean()
        return weights, indices


registry.register("router", "softmax_topk", lambda dim, num_experts, top_k, **kw: SoftmaxTopKRouter(dim, num_experts, top_k))
registry.register("router", "sigmoid_topk", lambda dim, num_experts, top_k, **kw: SigmoidTopKRouter(dim, num_experts, top_k, **kw))


def build_router(router_type: str, dim: int, num_experts: int, top_k: int, **kwargs) -> nn.Module:
    return registry.get("router", router_type)(dim, num_experts, top_k, **kwargs)
