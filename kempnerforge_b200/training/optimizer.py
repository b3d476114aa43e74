"""Optimizers: AdamW (fused over flat buffers), Lion, Schedule-Free AdamW, Muon.

``build_optimizer`` makes two parameter groups (weight decay for tensors with
more than one dimension whose name has no "bias", none for the rest) and hands
them to the builder registered under ``config.name``.

When the model's parameters live in flat buffers (``FlatParamGroup``), AdamW
updates a whole group — parameters, gradients and both moments — with one
kernel launch; the per-parameter ``state`` entries are views into the flat
moment buffers, so ``get_optimizer_state_dict`` / DCP still see
``exp_avg`` / ``exp_avg_sq`` / ``step`` under every parameter name.

Parity: kempnerforge/training/optimizer.py:28-589 — AdamW(lr, betas, eps; groups carry
the decay), Lion (sign of interpolated momentum, decoupled decay), Schedule-Free AdamW
(z / x / v iterates, internal warm-up, ``eval_params`` / ``train_params``, extra ``_k``),
Muon (momentum buffer, quintic Newton-Schulz on the local shard, sqrt(max(1, m/n)) scale,
inner AdamW for ineligible tensors whose LR follows Muon's LR ratio), eligibility
(>= 2-D, aspect ratio <= 10 after flattening trailing dims).
"""

from __future__ import annotations

import logging
import math

import torch

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.sections import OptimizerConfig
from kempnerforge_b200.ops import ref

log = logging.getLogger(__name__)


def _native():
    from kempnerforge_b200.ops import cuda as kc

    return kc


def _local(t: torch.Tensor) -> torch.Tensor:
    """Local shard of a DTensor, or the tensor itself."""
    return t.to_local() if hasattr(t, "to_local") else t


# --------------------------------------------------------------------------- AdamW
class FusedAdamW(torch.optim.AdamW):
    """``torch.optim.AdamW`` numerics; flat parameter groups update with one native launch each."""

    def __init__(self, params, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, fused=True):
        use_torch_fused = bool(fused) and torch.cuda.is_available()
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         fused=use_torch_fused or None)
        self._flat_groups: list = []
        self.grad_scale: torch.Tensor | None = None  # device scalar multiplied into every gradient
        self.skip_flag: torch.Tensor | None = None  # device int: non-zero turns the step into a no-op

    def attach_flat_groups(self, groups) -> None:
        """Register flat buffers; their parameters are then updated by the fused kernel only."""
        self._flat_groups = list(groups)
        for fg in self._flat_groups:
            fg.ensure_optimizer_state(self)

    @torch.no_grad()
    def step(self, closure=None):
        if not self._flat_groups:
            return super().step(closure)
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        from kempnerforge_b200.ops import cuda as kcuda

        lr = self.param_groups[0]["lr"]
        b1, b2 = self.param_groups[0]["betas"]
        eps = self.param_groups[0]["eps"]
        wd = max(g["weight_decay"] for g in self.param_groups)
        eng = getattr(self, "_engine", None)
        if eng is not None and eng.publish_on_side_stream(self._flat_groups):
            # sharded update + publication of every unit on the communication stream, in the order the next forward
            # pass needs them; each unit's forward waits for its own publication only
            def launch(fg):
                fg.step_count += 1
                p, g, m, v = fg.optimizer_views()
                if fg.world > 1:
                    lo, hi = fg.shard_range
                    kcuda.symm_adamw_bcast(fg.param_symm, g, m, v, lo, hi - lo, fg.n_decay, lr, b1, b2, eps, wd,
                                           fg.step_count, self.grad_scale, self.skip_flag)
                else:  # one GPU: the same ordering, without publication
                    kcuda.adamw_flat(p, g, m, v, fg.n_decay_local, lr, b1, b2, eps, wd, fg.step_count,
                                     self.grad_scale, self.skip_flag)

            for fg in self._flat_groups:
                fg.step_tensor.fill_(float(fg.step_count + 1))
            eng.publish_in_forward_order(launch)
            return loss
        for fg in self._flat_groups:
            fg.step_count += 1
            fg.step_tensor.fill_(float(fg.step_count))
            p, g, m, v = fg.optimizer_views()
            if p.numel() == 0:
                continue
            if p.is_cuda and getattr(fg, "param_symm", None) is not None and fg.world > 1:
                # sharded update fused with the parameter all-gather: new values go straight to every rank
                lo, hi = fg.shard_range
                kcuda.symm_adamw_bcast(fg.param_symm, g, m, v, lo, hi - lo, fg.n_decay, lr, b1, b2, eps, wd,
                                       fg.step_count, self.grad_scale, self.skip_flag)
            elif p.is_cuda:
                kcuda.adamw_flat(p, g, m, v, fg.n_decay_local, lr, b1, b2, eps, wd, fg.step_count,
                                 self.grad_scale, self.skip_flag)
            else:
                if self.grad_scale is not None:
                    g = g * self.grad_scale.to(g.dtype)
                nd = fg.n_decay_local
                ref.adamw_step_(p[:nd], g[:nd], m[:nd], v[:nd], fg.step_count, lr, b1, b2, eps, wd)
                ref.adamw_step_(p[nd:], g[nd:], m[nd:], v[nd:], fg.step_count, lr, b1, b2, eps, 0.0)
        return loss


@registry.register("optimizer", "adamw")
def _build_adamw(param_groups, config: OptimizerConfig):
    return FusedAdamW(param_groups, lr=config.lr, betas=tuple(config.betas), eps=config.eps, fused=config.fused)


# --------------------------------------------------------------------------- Lion
class Lion(torch.optim.Optimizer):
    """Sign-momentum optimizer: one state tensor (``exp_avg``) per parameter."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        if lr <= 0:
            raise ValueError(f"Invalid lr: {lr}")
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, (b1, b2), wd = group["lr"], group["betas"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if "exp_avg" not in state:
                    state["exp_avg"] = torch.zeros_like(p)
                pl, gl, ml = _local(p), _local(p.grad), _local(state["exp_avg"])
                if pl.is_cuda and _native().lion_step(pl, gl, ml, lr, b1, b2, wd):
                    continue  # one fused kernel did the update
                direction = torch.lerp(gl.to(ml.dtype), ml, b1).sign_()
                if wd:
                    pl.mul_(1.0 - lr * wd)
                pl.add_(direction.to(pl.dtype), alpha=-lr)
                ml.lerp_(gl.to(ml.dtype), 1.0 - b2)
        return loss


@registry.register("optimizer", "lion")
def _build_lion(param_groups, config: OptimizerConfig):
    return Lion(param_groups, lr=config.lr, betas=tuple(config.betas))


# --------------------------------------------------------------------------- Schedule-Free AdamW
class ScheduleFreeAdamW(torch.optim.Optimizer):
    """Schedule-free AdamW: gradient point y = lerp(z, x, beta1); x is the running average used for eval."""

    def __init__(self, params, lr=0.025, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, warmup_steps=0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.warmup_steps = warmup_steps
        self._k = 0

    def state_dict(self) -> dict:
        sd = super().state_dict()
        sd["_k"] = self._k
        sd["_warmup_steps"] = self.warmup_steps
        return sd

    def load_state_dict(self, state_dict: dict) -> None:
        state_dict = dict(state_dict)
        self._k = state_dict.pop("_k", self._k)
        self.warmup_steps = state_dict.pop("_warmup_steps", self.warmup_steps)
        super().load_state_dict(state_dict)
        # the step counter is not part of the per-parameter state that DCP carries; recover it
        for st in self.state.values():
            if "k" in st:
                self._k = max(self._k, int(st["k"]))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._k += 1
        k = self._k
        ramp = min(1.0, k / self.warmup_steps) if self.warmup_steps > 0 else 1.0
        for group in self.param_groups:
            lr = group["lr"] * ramp
            b1, b2 = group["betas"]
            eps, wd = group["eps"], group["weight_decay"]
            w_k = lr * (1.0 - b1)
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "z" not in st:
                    st["z"] = p.detach().clone()
                    st["v"] = torch.zeros_like(p)
                    st["weight_sum"] = 0.0
                z, v, g = _local(st["z"]), _local(st["v"]), _local(p.grad)
                if z.is_cuda:
                    first = "x" not in st
                    if first:
                        st["x"] = torch.empty_like(st["z"])
                    wsum = float(st["weight_sum"]) + w_k
                    if _native().sf_adamw_step(_local(p), g, z, v, _local(st["x"]), lr, b1, b2, eps, wd, 1.0 - b2**k,
                                               w_k / wsum, first):
                        st["weight_sum"], st["k"] = wsum, k
                        continue
                    if first:
                        del st["x"]
                v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
                z.addcdiv_(g, (v / (1.0 - b2**k)).sqrt_().add_(eps), value=-lr)
                if wd > 0:
                    z.mul_(1.0 - lr * wd)
                st["weight_sum"] = float(st["weight_sum"]) + w_k
                st["k"] = k
                if "x" not in st:
                    st["x"] = st["z"].clone()
                else:
                    _local(st["x"]).lerp_(z, w_k / st["weight_sum"])
                _local(p).copy_(z).lerp_(_local(st["x"]), b1)
        return loss

    @torch.no_grad()
    def eval_params(self) -> None:
        """Move parameters to the averaged iterate x (call before evaluation)."""
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state.get(p, {})
                if "x" in st:
                    _local(p).copy_(_local(st["x"]))

    @torch.no_grad()
    def train_params(self) -> None:
        """Move parameters back to the gradient point y = lerp(z, x, beta1)."""
        for group in self.param_groups:
            b1 = group["betas"][0]
            for p in group["params"]:
                st = self.state.get(p, {})
                if "z" in st and "x" in st:
                    _local(p).copy_(_local(st["z"])).lerp_(_local(st["x"]), b1)


@registry.register("optimizer", "schedule_free_adamw")
def _build_sf(param_groups, config: OptimizerConfig):
    return ScheduleFreeAdamW(param_groups, lr=config.lr, betas=tuple(config.betas), eps=config.eps,
                             warmup_steps=config.schedule_free_warmup_steps)


# --------------------------------------------------------------------------- Muon
def _newton_schulz_native(g: torch.Tensor, steps: int) -> torch.Tensor | None:
    """bf16 result of the iteration on the tcgen05 kernels, or None when the shape / device is not served.

    Per iteration: the Gram matrix A on the short side as a symmetric product (upper-triangle tiles only), the quintic
    aI + bA + cA^2 as a second symmetric product whose epilogue adds bA and the diagonal, and one GEMM that applies the
    polynomial to X; no elementwise pass in between.  The input may be bf16 or fp32; it is normalised in one pass.
    """
    if not (g.is_cuda and g.dim() == 2 and g.shape[0] % 8 == 0 and g.shape[1] % 8 == 0 and min(g.shape) >= 64):
        return None
    from kempnerforge_b200.ops import cuda as kcuda

    if not kcuda.available():
        return None
    a, b, c = ref.NS_COEFFS
    inv = 1.0 / (torch.linalg.vector_norm(g, dtype=torch.float32) + 1e-7)
    x = (g * inv).to(torch.bfloat16).contiguous()
    tall = x.shape[0] > x.shape[1]
    n = min(x.shape)
    symm = kcuda.gemm_symm_supported(x, tall)
    eye_a = None
    for _ in range(steps):
        if symm:
            gram = kcuda.gemm_symm(x, tall)                                         # A = X X^T or X^T X, symmetric
            poly = kcuda.gemm_symm(gram, False, residual=gram, alpha=c, beta=b, diag=a)   # aI + bA + cA^2
        else:
            if eye_a is None:
                eye_a = torch.zeros(n, n, dtype=torch.float32, device=x.device)
                eye_a.diagonal().fill_(a)
            gram = kcuda.gemm(x, x, a_kmajor=False, b_kmajor=False) if tall else kcuda.gemm(x, x)
            sq = kcuda.gemm(gram, gram, out_dtype=torch.float32)
            poly = (eye_a + b * gram.float() + c * sq).to(torch.bfloat16)
        x = kcuda.gemm(x, poly) if tall else kcuda.gemm(poly, x, b_kmajor=False)
    return x


def newton_schulz(g: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation (fp32 out).

    On CUDA every iteration is three bf16 tcgen05 GEMMs with fp32 accumulation.  The Gram matrix is always taken
    on the short side: X' = (aI + bA + cA^2) X with A = X X^T for a wide X, and X' = X (aI + bA + cA^2) with
    A = X^T X for a tall one.  Both are the same polynomial in X (X X^T X = X (X^T X)), so the result is the one the
    un-transposed formulation gives, at min(m, n)^2 max(m, n) instead of max(m, n)^2 min(m, n) flops per product;
    the ``a X`` term rides on the diagonal of the polynomial, so the last GEMM writes the next iterate directly.
    Elsewhere (CPU, odd shapes) the plain fp32 formulation runs.
    """
    x = _newton_schulz_native(g, steps)
    return x.float() if x is not None else ref.newton_schulz(g, steps)


_newton_schulz = newton_schulz


def is_muon_eligible(p: torch.Tensor) -> bool:
    if p.dim() < 2:
        return False
    rows, cols = p.shape[0], p.numel() // max(1, p.shape[0])
    return max(rows, cols) / max(1, min(rows, cols)) <= 10


_is_muon_eligible = is_muon_eligible   # underscore spelling used by code written against the reference


class Muon(torch.optim.Optimizer):
    """Momentum + Newton-Schulz orthogonalised updates for matrices; AdamW for everything else."""

    def __init__(self, muon_params, adam_params, lr=0.02, momentum=0.95, weight_decay=0.0,
                 adam_betas=(0.9, 0.95), adam_eps=1e-8, ns_steps=5, adam_lr=None):
        adam_lr = lr if adam_lr is None else adam_lr
        self._initial_lr = lr
        self._initial_adam_lr = adam_lr
        has_adam = any(len(g["params"]) for g in adam_params)
        self._adam = FusedAdamW(adam_params, lr=adam_lr, betas=adam_betas, eps=adam_eps) if has_adam else None
        # data-parallel group over which the Newton-Schulz work is divided (set by build_optimizer; None = every rank
        # orthogonalises every matrix, like the reference)
        self.dp_group = None
        super().__init__(muon_params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, ns_steps=ns_steps))

    @property
    def inner_adam(self):
        return self._adam

    def state_dict(self) -> dict:
        sd = super().state_dict()
        if self._adam is not None:
            sd["_adam_state"] = self._adam.state_dict()
        sd["_initial_lr"] = self._initial_lr
        sd["_initial_adam_lr"] = self._initial_adam_lr
        return sd

    def load_state_dict(self, state_dict: dict) -> None:
        state_dict = dict(state_dict)
        adam_state = state_dict.pop("_adam_state", None)
        self._initial_lr = state_dict.pop("_initial_lr", self._initial_lr)
        self._initial_adam_lr = state_dict.pop("_initial_adam_lr", self._initial_adam_lr)
        super().load_state_dict(state_dict)
        if adam_state is not None and self._adam is not None:
            self._adam.load_state_dict(adam_state)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        import torch.distributed as dist

        dp = self.dp_group
        world = dist.get_world_size(dp) if dp is not None else 1
        rank = dist.get_rank(dp) if dp is not None else 0
        pending = []   # (work handle) of parameter broadcasts in flight
        k = 0          # running index of non-empty matrices: matrix k is orthogonalised by data-parallel rank k % world
        for group in self.param_groups:
            lr, mu, wd, ns = group["lr"], group["momentum"], group["weight_decay"], group["ns_steps"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p.grad)
                pl, gl, buf = _local(p), _local(p.grad), _local(st["momentum_buffer"])
                buf.mul_(mu).add_(gl)   # every rank keeps every momentum buffer (the gradients are identical)
                if buf.numel() == 0:
                    continue
                owner = k % world
                k += 1
                if owner == rank:
                    mat = buf.reshape(buf.shape[0], -1)
                    shape_scale = math.sqrt(max(1.0, mat.shape[0] / mat.shape[1]))
                    if wd > 0:
                        pl.mul_(1.0 - lr * wd)
                    upd = _newton_schulz_native(mat, ns)
                    if upd is not None:   # bf16 iterate straight into the parameter: one pass, one rounding
                        pl.add_(upd.view_as(pl), alpha=-lr * shape_scale)
                    else:
                        upd = newton_schulz(mat.float(), ns).mul_(shape_scale)
                        pl.add_(upd.to(pl.dtype).view_as(pl), alpha=-lr)
                if world > 1:
                    # the owner's new values replace everybody's copy; the transfer overlaps the next matrices' math
                    src = dist.get_global_rank(dp, owner)
                    pending.append(dist.broadcast(pl if pl.is_contiguous() else pl.data, src=src, group=dp, async_op=True))
        for work in pending:
            work.wait()
        if self._adam is not None:
            if self._initial_lr > 0:
                ratio = self.param_groups[0]["lr"] / self._initial_lr
                for g in self._adam.param_groups:
                    g["lr"] = self._initial_adam_lr * ratio
            self._adam.step()
        return loss


@registry.register("optimizer", "muon")
def _build_muon(param_groups, config: OptimizerConfig):
    muon_groups, adam_groups = [], []
    for group in param_groups:
        rest = {k: v for k, v in group.items() if k != "params"}
        elig = [p for p in group["params"] if is_muon_eligible(p)]
        other = [p for p in group["params"] if not is_muon_eligible(p)]
        if elig:
            muon_groups.append({**rest, "params": elig})
        if other:
            adam_groups.append({**rest, "params": other})
    if not adam_groups:
        adam_groups = [{"params": [], "weight_decay": 0.0}]
    log.info(
        "Muon: %s params (NS-orthogonalized), %s params (AdamW fallback)",
        f"{sum(p.numel() for g in muon_groups for p in g['params']):,}",
        f"{sum(p.numel() for g in adam_groups for p in g['params']):,}",
    )
    return Muon(muon_groups, adam_groups, lr=config.lr, momentum=config.muon_momentum,
                weight_decay=config.weight_decay, adam_betas=tuple(config.betas), adam_eps=config.eps,
                ns_steps=config.muon_ns_steps, adam_lr=config.muon_adam_lr)


# --------------------------------------------------------------------------- groups
def should_decay(name: str, param: torch.Tensor) -> bool:
    return param.dim() > 1 and "bias" not in name


_should_decay = should_decay


def build_param_groups(model: torch.nn.Module, weight_decay: float) -> list[dict]:
    decay, no_decay = [], []
    for name, p in model.named_parameters():
        if p.requires_grad:
            (decay if should_decay(name, p) else no_decay).append(p)
    log.info(
        "Optimizer groups: %s params with decay, %s params without decay",
        f"{sum(p.numel() for p in decay):,}", f"{sum(p.numel() for p in no_decay):,}",
    )
    return [{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}]


def build_optimizer(model: torch.nn.Module, config: OptimizerConfig) -> torch.optim.Optimizer:
    groups = build_param_groups(model, config.weight_decay)
    opt = registry.get("optimizer", config.name)(groups, config)
    flat = getattr(model, "_kf_flat_groups", None)
    if flat and isinstance(opt, FusedAdamW):
        opt.attach_flat_groups(flat)
        opt._engine = getattr(model, "_kf_engine", None)
    elif getattr(getattr(model, "_kf_engine", None), "shard_blocks", False):
        raise ValueError(f"optimizer {config.name!r} steps on whole parameters; sharded parameters (ZeRO-3) need adamw "
                         "(set distributed param sharding to 'resident' for the other optimizers)")
    elif getattr(model, "_kf_engine", None) is not None:
        # whole-parameter optimizers read every element of ``p.grad``: the engine must leave the complete averaged
        # gradient on every rank, not only the local shard of each flat buffer
        model._kf_engine.full_grads = True
        if isinstance(opt, Muon) and model._kf_engine.world > 1:
            opt.dp_group = model._kf_engine.pg   # divide the Newton-Schulz work over the data-parallel ranks
    if getattr(model, "_kf_engine", None) is not None:
        model._kf_engine.bind_optimizer(opt)     # plain backward / step / zero_grad loops work without engine calls
    return opt
