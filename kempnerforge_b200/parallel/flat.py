"""Flat parameter storage.

A ``FlatParamGroup`` owns one contiguous buffer for the parameters of one unit
(a transformer block, or the root unit: embedding + final norm + head), a
same-shaped gradient buffer and — once an optimizer attaches — flat moment
buffers.  Every ``nn.Parameter`` of the unit becomes a view into the buffer, so

* adjacent projection weights (q|k|v, gate|up) form one GEMM operand without a copy,
* weight-gradient GEMMs write straight into the flat gradient buffer,
* the optimizer updates the whole unit with one kernel launch,
* data-parallel reduction / broadcast work on one address range per unit
  (the buffers can be placed in NVLink symmetric memory by passing an allocator).

Layout: parameters that get weight decay first, then the rest, each aligned to
16 bytes; under data parallelism the flat range is cut into ``world`` equal
shards (optimizer state exists only for the local shard).

Replaces what FSDP2's ``fully_shard`` does for the reference
(kempnerforge/distributed/parallel.py:216-302): unit = one block, root unit =
embedding + norm + head, parameters in the training dtype, gradients averaged
over the data-parallel group.
"""

from __future__ import annotations

from collections.abc import Callable, Iterable

import torch
from torch import nn

ALIGN_BYTES = 16


def _should_decay(name: str, p: torch.Tensor) -> bool:
    return p.dim() > 1 and "bias" not in name


class FlatParamGroup:
    def __init__(
        self,
        name: str,
        named_params: Iterable[tuple[str, nn.Parameter]],
        world: int = 1,
        rank: int = 0,
        allocator: Callable[[int, torch.dtype, torch.device], torch.Tensor] | None = None,
        local: bool = False,
        sharded: bool = False,
    ) -> None:
        """``sharded=True`` (ZeRO-3): this rank keeps only piece ``rank`` of every parameter (``self.shard``, the
        pieces packed in parameter order) plus the matching gradient shard and moments; the whole parameters and
        gradients exist only in staging buffers that the engine binds with :meth:`bind` and that are shared by all
        units.  Every parameter is padded to a multiple of ``8 * world`` elements so that all pieces are 16-byte
        aligned and equally long — per-parameter dim-0 sharding like ``fully_shard`` of the reference
        (kempnerforge/distributed/parallel.py:250-302), which keeps every rank's NVLink egress equal when a weight
        is gathered."""
        self.name = name
        self.sharded = bool(sharded) and world > 1 and not local
        # a "local" group holds parameters that exist only on this rank (expert-parallel experts inside the
        # data-parallel group): it is neither reduced nor sharded across the data-parallel ranks
        self.local = local
        if local:
            world, rank = 1, 0
        self.world, self.rank = world, rank
        items = [(n, p) for n, p in named_params if p.requires_grad]
        if not items:
            raise ValueError(f"flat group {name!r} has no trainable parameters")
        self.dtype = items[0][1].dtype
        self.device = items[0][1].device
        if any(p.dtype != self.dtype or p.device != self.device for _, p in items):
            raise ValueError(f"flat group {name!r} mixes dtypes or devices")
        elem = torch.empty((), dtype=self.dtype).element_size()
        align = max(1, ALIGN_BYTES // elem) * (world if self.sharded else 1)
        decay = [(n, p) for n, p in items if _should_decay(n, p)]
        rest = [(n, p) for n, p in items if not _should_decay(n, p)]
        # tensor-parallel shards first: their squared norm has to be summed over the TP group, while the
        # replicated tensors behind the boundary count once (a stable partition keeps q|k|v and gate|up adjacent)
        is_tp = lambda p: getattr(p, "_kf_shard", ("", 0))[0] == "tp"  # noqa: E731
        n_tp_params = sum(1 for _, p in decay if is_tp(p))
        decay = [x for x in decay if is_tp(x[1])] + [x for x in decay if not is_tp(x[1])]
        self.names: list[str] = []
        self.params: list[nn.Parameter] = []
        self.offsets: list[int] = []
        off = 0
        for n, p in decay + rest:
            self.names.append(n)
            self.params.append(p)
            self.offsets.append(off)
            off += -(-p.numel() // align) * align
        self.n_decay = self.offsets[len(decay)] if rest else off
        if not decay:
            self.n_decay = 0
        all_items = decay + rest
        self.n_tp_sharded = (self.offsets[n_tp_params] if n_tp_params < len(all_items) else off) if n_tp_params else 0
        self.ep_sharded = False  # set by flatten_model for expert groups of an expert-parallel model
        # pad so that every rank's shard has the same, aligned length
        chunk = align * world
        self.numel = -(-off // chunk) * chunk
        self.shard_numel = self.numel // world
        alloc = allocator or (lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev))
        if self.sharded:
            self._init_sharded(alloc, allocator is not None)
            return
        self.param = alloc(self.numel, self.dtype, self.device)
        self.grad = alloc(self.numel, self.dtype, self.device)
        # symmetric-memory descriptors of the two buffers (None with an ordinary allocator)
        self.param_symm = self.grad_symm = None
        if allocator is not None and not local:
            from kempnerforge_b200.comm import symmetric

            self.param_symm = symmetric.lookup(self.param)
            self.grad_symm = symmetric.lookup(self.grad)
        self.exp_avg: torch.Tensor | None = None
        self.exp_avg_sq: torch.Tensor | None = None
        self.step_tensor = torch.zeros((), dtype=torch.float32)
        self.step_count = 0
        with torch.no_grad():
            for p, o in zip(self.params, self.offsets):
                view = self.param[o : o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p._kf_grad = self.grad[o : o + p.numel()].view(p.shape)
                p._kf_grad_live = False
                p._kf_flat = self

    # ------------------------------------------------------------------ sharded parameters (ZeRO-3)
    def _init_sharded(self, alloc, symmetric: bool) -> None:
        w, r = self.world, self.rank
        # padded length of every parameter = distance to the next offset
        ends = self.offsets[1:] + [self.numel]
        self.padded = [e - o for o, e in zip(self.offsets, ends)]
        self.shard = alloc(self.shard_numel, self.dtype, self.device)          # this rank's piece of every parameter
        self.grad_shard = torch.zeros(self.shard_numel, dtype=self.dtype, device=self.device)
        self.grad_shard_live = False
        self.shard_symm = None
        if symmetric:
            from kempnerforge_b200.comm import symmetric as symm

            self.shard_symm = symm.lookup(self.shard)
        self.param = self.grad = None        # whole buffers exist only while bound to staging
        self.param_symm = self.grad_symm = None
        self.grad_stage_symm = None
        self.valid: set = set()              # which parts of the bound parameter staging hold this unit's current values
        self.engine = None
        self.exp_avg = self.exp_avg_sq = None
        self.step_tensor = torch.zeros((), dtype=torch.float32)
        self.step_count = 0
        with torch.no_grad():
            for p, o, n in zip(self.params, self.offsets, self.padded):
                piece = n // w
                flat = p.data.reshape(-1)
                lo, hi = r * piece, min((r + 1) * piece, flat.numel())
                dst = self.shard[o // w : o // w + piece]
                dst.zero_()
                if hi > lo:
                    dst[: hi - lo].copy_(flat[lo:hi])
                p._kf_flat = self
                p._kf_grad_live = False

    def piece_of(self, p) -> torch.Tensor:
        """This rank's piece of parameter ``p`` inside the shard (1-D, padded length / world)."""
        i = next(k for k, q in enumerate(self.params) if q is p)
        return self.shard[self.offsets[i] // self.world : (self.offsets[i] + self.padded[i]) // self.world]

    def index_of(self, p) -> int:
        return next(k for k, q in enumerate(self.params) if q is p)

    def bind(self, param_stage: torch.Tensor, grad_stage: torch.Tensor | None, grad_stage_symm=None) -> None:
        """Point the unit's parameters (and gradient slots) at staging buffers.  The contents are whatever the
        staging holds: the engine pulls the current values before they are read."""
        self.param = param_stage[: self.numel]
        self.grad = grad_stage[: self.numel] if grad_stage is not None else None
        self.grad_stage_symm = grad_stage_symm
        for p, o in zip(self.params, self.offsets):
            p.data = self.param[o : o + p.numel()].view(p.shape)
            if self.grad is not None:
                p._kf_grad = self.grad[o : o + p.numel()].view(p.shape)

    # ------------------------------------------------------------------ shards
    @property
    def shard_range(self) -> tuple[int, int]:
        lo = self.rank * self.shard_numel
        return lo, lo + self.shard_numel

    @property
    def n_decay_local(self) -> int:
        """Number of leading elements of the local shard that receive weight decay."""
        if self.sharded:
            return self.n_decay // self.world
        lo, hi = self.shard_range
        return max(0, min(self.n_decay, hi) - lo)

    def optimizer_views(self):
        """(param shard, grad shard, exp_avg, exp_avg_sq) for the local rank."""
        if self.sharded:
            return self.shard, self.grad_shard, self.exp_avg, self.exp_avg_sq
        lo, hi = self.shard_range
        return self.param[lo:hi], self.grad[lo:hi], self.exp_avg, self.exp_avg_sq

    # ------------------------------------------------------------------ gradients
    def zero_grad(self) -> None:
        """Forget accumulated gradients; the buffer itself is overwritten by the next backward."""
        if self.sharded:
            self.grad_shard_live = False
        for p in self.params:
            p._kf_grad_live = False
            p.grad = None

    def finalize_grads(self) -> None:
        """Make the flat buffer hold every gradient: fold in autograd-produced ``.grad`` tensors, zero
        the slots nothing wrote, and point ``.grad`` at the flat views."""
        if self.sharded and getattr(self.engine, "shared_staging", True):
            return  # gradients went through the shared staging buffer and were reduced into the shard block by block
        with torch.no_grad():
            for p in self.params:
                slot = p._kf_grad
                g = p.grad
                if g is not None and g.data_ptr() != slot.data_ptr():
                    g = g.to_local() if hasattr(g, "to_local") else g
                    if p._kf_grad_live:
                        slot.add_(g.to(slot.dtype))
                    else:
                        slot.copy_(g)
                    p._kf_grad_live = True
                elif g is None and not p._kf_grad_live:
                    slot.zero_()
                p.grad = slot

    # ------------------------------------------------------------------ optimizer state
    def ensure_optimizer_state(self, optimizer: torch.optim.Optimizer, state_dtype: torch.dtype | None = None) -> None:
        """Allocate flat moments for the local shard and expose per-parameter views in ``optimizer.state``.

        With world == 1 the views cover whole parameters, so the state dict is exactly what
        ``torch.optim.AdamW`` would hold.  With world > 1 the per-parameter entries are created on
        demand by ``full_optimizer_state`` (checkpointing) instead.
        """
        dt = state_dtype or self.dtype
        if self.exp_avg is None:
            self.exp_avg = torch.zeros(self.shard_numel, dtype=dt, device=self.device)
            self.exp_avg_sq = torch.zeros(self.shard_numel, dtype=dt, device=self.device)
            self.step_tensor = torch.zeros((), dtype=torch.float32, device=self.device)
        if self.world == 1:
            for p, o in zip(self.params, self.offsets):
                optimizer.state[p] = {
                    "step": self.step_tensor,
                    "exp_avg": self.exp_avg[o : o + p.numel()].view(p.shape),
                    "exp_avg_sq": self.exp_avg_sq[o : o + p.numel()].view(p.shape),
                }

    def load_step(self, step: int) -> None:
        self.step_count = int(step)
        self.step_tensor.fill_(float(step))


def group_module_params(module: nn.Module, prefix: str = "") -> list[tuple[str, nn.Parameter]]:
    seen, out = set(), []
    for n, p in module.named_parameters():
        if id(p) in seen:
            continue
        seen.add(id(p))
        out.append((prefix + n, p))
    return out


def flatten_model(model: nn.Module, world: int = 1, rank: int = 0, allocator=None,
                  shard_blocks: bool = False) -> list[FlatParamGroup]:
    """One flat group per transformer block plus a root group for everything else.

    Returns the groups in forward order (root group last) and records them on the model.
    """
    groups: list[FlatParamGroup] = []
    taken: set[int] = set()
    ep_local = bool(getattr(model, "ep_in_dp", False))

    has_ep = getattr(model, "ep_group", None) is not None

    def is_local(p) -> bool:
        return has_ep and (getattr(p, "_kf_ep_local", False) or getattr(p, "_kf_shard", ("", 0))[0] == "ep")

    def add(name: str, items) -> None:
        items = [(n, p) for n, p in items if id(p) not in taken and p.requires_grad]
        shared = [(n, p) for n, p in items if not is_local(p)]
        mine = [(n, p) for n, p in items if is_local(p)]
        if shared:
            groups.append(FlatParamGroup(name, shared, world, rank, allocator,
                                         sharded=shard_blocks and name != "root" and not name.startswith("root.")))
        if mine:
            groups.append(FlatParamGroup(name + ".experts", mine, world, rank, None if ep_local else allocator, local=ep_local))
            groups[-1].ep_sharded = True
        taken.update(id(p) for _, p in items)

    # the block stack may sit below a wrapper (vision-language models): use the first ``layers`` ModuleDict
    for mod_name, mod in model.named_modules():
        layers = getattr(mod, "layers", None)
        if isinstance(layers, nn.ModuleDict):
            base = f"{mod_name}.layers" if mod_name else "layers"
            for key, block in layers.items():
                add(f"{base}.{key}", group_module_params(block, f"{base}.{key}."))
            break
    by_dtype: dict[torch.dtype, list] = {}
    for n, p in group_module_params(model):
        if id(p) not in taken and p.requires_grad:
            by_dtype.setdefault(p.dtype, []).append((n, p))
    for i, (dt, items) in enumerate(by_dtype.items()):
        add("root" if i == 0 else f"root.{i}", items)
    model._kf_flat_groups = groups
    return groups
