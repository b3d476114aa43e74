"""Sharded data-parallel engine over flat parameter groups.

Memory plan ("resident" ZeRO): every rank keeps the full bf16 parameters and a full
gradient buffer of each unit — on a 180 GB part an 8 B-parameter model needs 32 GB for
both — while optimizer state and the optimizer work are sharded 1/N.  A training step is

  backward  -> flat gradient buffers (local sum over micro-batches)
  reduce    -> every rank obtains the mean gradient of *its* shard (reduce-scatter)
  clip      -> global norm from the shard sums of squares (one scalar all-reduce, no host sync)
  update    -> fused AdamW on the shard
  publish   -> the updated shard is written into every rank's parameter buffer (all-gather)

Two transports implement reduce/publish:
  * ``collective``: ``torch.distributed`` calls (NCCL on GPUs, gloo on CPU) — the portable baseline;
  * ``symmetric``: our own kernels over NVLink symmetric memory (see ``kempnerforge_b200.comm``),
    where the reduce-scatter is fused with the scaling / cast / norm partial and the
    all-gather is fused into the AdamW kernel's stores.

Gradient accumulation: ``set_requires_gradient_sync(False)`` marks a micro-step after which
nothing is reduced (kempnerforge/training/grad.py:15-39).  Gradient clipping mirrors
kempnerforge/distributed/utils.py:44-111: coef = max_norm / (norm + 1e-6) clamped to 1, the
pre-clip norm is returned.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch import nn

from kempnerforge_b200.parallel.flat import FlatParamGroup, flatten_model


class DataParallelEngine:
    def __init__(self, model: nn.Module, process_group=None, transport: str = "collective", allocator=None) -> None:
        self.model = model
        self.pg = process_group
        self.world = dist.get_world_size(process_group) if process_group is not None else 1
        self.rank = dist.get_rank(process_group) if process_group is not None else 0
        self.transport = transport
        self.groups: list[FlatParamGroup] = flatten_model(model, self.world, self.rank, allocator,
                                                          shard_blocks=bool(getattr(self, "shard_blocks", False)))
        self.requires_sync = True
        dev = self.groups[0].device
        self.device = dev
        self._sq3 = torch.zeros(3, dtype=torch.float32, device=dev)
        self.grad_scale = torch.ones(1, dtype=torch.float32, device=dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self._reduced = False
        self._manual_step = False    # this step's gradient reduction was started by an optimizer / clipping hook
        self._expose_queued = False  # an end-of-backward callback is already queued for the running backward pass
        self._scale_pending = False  # a clip factor was computed and not yet multiplied into whole gradients
        self._reduce_work: dict[int, object] = {}  # group index -> in-flight gradient reduction
        self._gather_work: dict[int, object] = {}  # group index -> in-flight parameter publication
        self._group_of_module: dict[int, int] = {}
        self._handles: list = []   # forward pre-hooks installed on the model
        self._wrapped: list[str] = []  # model methods replaced by waiting wrappers
        self.symmetric = transport == "symmetric" and self.world > 1 and any(
            getattr(g, "grad_symm", None) is not None or getattr(g, "shard_symm", None) is not None for g in self.groups)
        self._comm_stream = torch.cuda.Stream() if (self.symmetric and dev.type == "cuda") else None
        self._sq_from_reduce = False
        self._root_groups: list[int] = []
        self._published_per_group = False
        # True when the optimizer steps on whole parameters (Lion, Schedule-Free AdamW, Muon) instead of the flat
        # shards: every rank then needs the *whole* averaged gradient, not only its shard (set by build_optimizer)
        self.full_grads = False
        # library-collective path: reduce gradients in fp32 (KF_DP_REDUCE_DTYPE=bf16 trades that for half the traffic)
        self.reduce_fp32 = os.environ.get("KF_DP_REDUCE_DTYPE", "fp32").lower() in ("fp32", "float32")
        model._kf_engine = self
        model.set_requires_gradient_sync = self.set_requires_gradient_sync
        # One GPU: the flat AdamW of a step (bound by memory bandwidth) runs on a side stream, unit by unit in forward
        # order, under the next step's forward pass (bound by the tensor cores); a block waits for its own unit only.
        self.overlap_update = (self.world == 1 and dev.type == "cuda" and not getattr(self, "shard_blocks", False)
                               and os.environ.get("KF_DP_OVERLAP_UPDATE", "1") != "0")
        if self.overlap_update:
            self._comm_stream = torch.cuda.Stream()
            self._install_overlap_hooks()
        if self.world > 1:
            self.broadcast_parameters()
            self._install_overlap_hooks()
        # whatever the hooks above cover: a backward pass that starts from the model's output ends by presenting the
        # flat gradient slots as ``.grad`` (see queue_expose_flat_grads)
        self._aux_handles = [model.register_forward_hook(self._attach_expose)]

    # ------------------------------------------------------------------ set-up
    def broadcast_parameters(self, src: int = 0) -> None:
        """Make every rank start from rank ``src``'s weights."""
        root = dist.get_global_rank(self.pg, src) if self.pg is not None else src
        for g in self.groups:
            if g.local:
                continue
            dist.broadcast(g.param, src=root, group=self.pg)

    # ------------------------------------------------------------------ overlap of communication with compute
    def _install_overlap_hooks(self) -> None:
        """Reduce a block's gradients as soon as its backward finished, and wait for a block's freshly
        published parameters only when its forward starts."""
        by_name = {g.name: i for i, g in enumerate(self.groups)}
        covered: set[int] = set()
        for mod_name, mod in self.model.named_modules():  # the block stack may sit below a wrapper module
            layers = getattr(mod, "layers", None)
            if not isinstance(layers, nn.ModuleDict):
                continue
            base = f"{mod_name}.layers" if mod_name else "layers"
            for key, block in layers.items():
                idx = by_name.get(f"{base}.{key}")
                if idx is None:
                    continue
                extra = by_name.get(f"{base}.{key}.experts")
                idxs = [idx] + ([extra] if extra is not None else [])
                covered.update(idxs)
                self._handles.append(block.register_forward_pre_hook(self._make_pre_hook(idxs)))
            break
        # everything that no block hook covers is waited for when the model itself is entered
        root = [i for i in range(len(self.groups)) if i not in covered]
        self._root_groups = root
        self._handles.append(self.model.register_forward_pre_hook(lambda m, a: self.wait_params(root)))
        for name in ("forward_hidden", "compute_loss"):
            fn = getattr(self.model, name, None)
            if fn is not None:
                setattr(self.model, name, self._wrap_wait(fn, root))
                self._wrapped.append(name)

    def _wrap_wait(self, fn, idxs):
        def wrapped(*a, **k):
            self.wait_params(idxs)
            return fn(*a, **k)

        return wrapped

    def _make_pre_hook(self, idxs):
        def hook(module, args):
            self.wait_params(idxs)
            x = args[0] if args else None
            if torch.is_tensor(x) and x.requires_grad and torch.is_grad_enabled() and self.requires_sync:
                x.register_hook(lambda g, idxs=idxs: self._block_backward_done(idxs))

        return hook

    def wait_params(self, idxs) -> None:
        for i in idxs:
            work = self._gather_work.pop(i, None)
            if work is not None:
                work.wait()

    def _attach_expose(self, module, args, output) -> None:
        out = output[0] if isinstance(output, (tuple, list)) and output else output
        if torch.is_tensor(out) and out.requires_grad and torch.is_grad_enabled():
            out.register_hook(lambda grad: self.queue_expose_flat_grads())

    def queue_expose_flat_grads(self) -> None:
        """Called from inside a backward pass: when the pass ends, parameters whose gradient a fused node wrote straight
        into the flat buffer (autograd saw ``None`` for them) show that slot as ``.grad``, so code that looks at
        gradients between ``backward()`` and ``step()`` finds them where it expects them."""
        if not self._expose_queued:
            self._expose_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._expose_flat_grads)

    def _expose_flat_grads(self) -> None:
        self._expose_queued = False
        for g in self.groups:
            if getattr(g, "sharded", False):
                continue          # slots of sharded units live in a staging buffer that the next block reuses
            for p in g.params:
                if p.grad is not None or not p.requires_grad:
                    continue
                if not getattr(p, "_kf_grad_live", False):
                    # nothing reached this parameter in the pass (an unused branch): the optimizer's flat update
                    # treats it as a zero gradient, so that is what ``.grad`` shows
                    p._kf_grad.zero_()
                    p._kf_grad_live = True
                p.grad = p._kf_grad

    def _block_backward_done(self, idxs) -> None:
        self.queue_expose_flat_grads()
        if not (self.world > 1 and self.requires_sync):
            return None
        for i in idxs:
            g = self.groups[i]
            if i in self._reduce_work or g.local:
                continue
            ready = all(
                getattr(p, "_kf_grad_live", False) and (p.grad is None or p.grad.data_ptr() == p._kf_grad.data_ptr())
                for p in g.params
            )
            if not ready:
                continue
            tp = getattr(self.model, "tp", None)
            if tp is not None:  # gradients that only saw part of the tokens are summed over the TP group first
                from kempnerforge_b200.parallel.tensor_parallel import sync_partial_grads_of

                sync_partial_grads_of(g.params, tp)
            ep_group = getattr(self.model, "ep_group", None)
            if ep_group is not None and not getattr(self.model, "ep_in_dp", False) and g.ep_sharded:
                g.grad.div_(dist.get_world_size(ep_group))  # shared-batch EP: every expert saw each token once per peer
                g._kf_ep_scaled = True
            self._reduce_work[i] = self._reduce_one(g, async_op=True)
        return None

    def _reduce_one(self, g: FlatParamGroup, async_op: bool = False):
        if self.symmetric and g.grad_symm is not None:
            return self._reduce_one_symmetric(g, async_op)
        if g.grad.is_cuda and "nccl" in str(dist.get_backend(self.pg)):
            if self.full_grads:
                return dist.all_reduce(g.grad, op=dist.ReduceOp.AVG, group=self.pg, async_op=async_op)
            lo, hi = g.shard_range
            if self.reduce_fp32 and g.grad.dtype != torch.float32:
                # the sum over ranks is taken in fp32 and rounded once (what the peer-memory kernels do, and the
                # reduce_dtype of the mixed-precision policy); costs a transient fp32 copy of one unit
                wide = g.grad.float()
                out = torch.empty(hi - lo, dtype=torch.float32, device=g.grad.device)
                work = dist.reduce_scatter_tensor(out, wide, op=dist.ReduceOp.AVG, group=self.pg, async_op=async_op)
                if async_op:
                    return _CopyAfterWork(work, out, g.grad[lo:hi], wide)
                g.grad[lo:hi].copy_(out)
                return None
            return dist.reduce_scatter_tensor(g.grad[lo:hi], g.grad, op=dist.ReduceOp.AVG, group=self.pg, async_op=async_op)
        work = dist.all_reduce(g.grad, group=self.pg, async_op=async_op)
        if async_op:
            return _ScaledWork(work, g.grad, self.world)
        g.grad.div_(self.world)
        return None

    def _reduce_one_symmetric(self, g: FlatParamGroup, async_op: bool):
        """Barrier (all ranks finished writing this unit's gradients) + fused reduce-scatter / scale / norm
        kernel over peer memory; on the side stream when launched from a block's backward hook."""
        from kempnerforge_b200.ops import cuda as kcuda

        lo, hi = g.shard_range
        slot = 2 if g.ep_sharded else 0
        if not self._sq_from_reduce:
            self._sq3.zero_()
            self._sq_from_reduce = True

        def launch():
            g.grad_symm.barrier()
            kcuda.symm_rs_norm(g.grad_symm, lo, hi - lo, self._sq3[slot : slot + 1], accumulate=True)
            if self.full_grads:
                # whole-parameter optimizers: every rank also needs the other shards of the averaged gradient
                g.grad_symm.barrier()  # every rank has finished reading the un-averaged values of this range
                kcuda.symm_gather(g.grad_symm, lo, hi - lo)
                g.grad_symm.barrier()

        if not async_op or self._comm_stream is None:
            launch()
            return None
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ready)
            launch()
            done = torch.cuda.Event()
            done.record()
        return _EventWork(done)

    def set_requires_gradient_sync(self, flag: bool) -> None:
        self.requires_sync = bool(flag)

    # ------------------------------------------------------------------ step phases
    def finish_backward(self) -> None:
        """Fold stray autograd gradients into the flat buffers and reduce them across ranks."""
        for g in self.groups:
            g.finalize_grads()
        if getattr(self.model, "tp", None) is not None:
            from kempnerforge_b200.parallel.tensor_parallel import sync_partial_grads

            sync_partial_grads(self.model)
        ep_group = getattr(self.model, "ep_group", None)
        if ep_group is not None and not getattr(self.model, "ep_in_dp", False) and self.requires_sync:
            # EP peers route the *same* batch, so every expert saw each token once per peer: undo that factor
            ep = dist.get_world_size(ep_group)
            for g in self.groups:
                if g.ep_sharded and not getattr(g, "_kf_ep_scaled", False):
                    g.grad.div_(ep)
        if self.world > 1 and self.requires_sync:
            self._reduce_gradients()
        self._reduced = True

    def _reduce_gradients(self) -> None:
        for i, g in enumerate(self.groups):
            if g.local:  # rank-private parameters: the gradient is complete, only the loss averaging applies
                g.grad.div_(self.world)
                continue
            work = self._reduce_work.pop(i, None)
            if work is not None:  # already launched from the block's backward hook
                work.wait()
                continue
            self._reduce_one(g)

    def _sumsq_into(self, x: torch.Tensor, slot: int) -> None:
        if x.numel() == 0:
            return
        if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32):
            from kempnerforge_b200.ops import cuda as kcuda

            kcuda.sumsq(x, self._sq3[slot : slot + 1], accumulate=True)
        else:
            self._sq3[slot] += x.float().pow(2).sum()

    def clip_grad_norm(self, max_norm: float | None, extra_groups=()) -> torch.Tensor:
        """Global gradient L2 norm (pre-clip, device scalar); sets ``grad_scale`` for the optimizer.

        Squared sums are kept in three buckets: tensors replicated over the model-parallel groups, tensor-parallel
        shards (summed over the TP group) and expert-parallel shards (summed over the EP group).  Every bucket is
        first summed over the data-parallel shards; ``extra_groups`` (pipeline stages) are summed last.
        """
        if self._sq_from_reduce:  # the fused reduce kernels already produced the shard sums of squares
            self._sq_from_reduce = False
            if self.world > 1:
                dist.all_reduce(self._sq3, group=self.pg)
            total = self._sq3.sum().reshape(1)
            for grp in extra_groups:
                dist.all_reduce(total, group=grp)
            torch.sqrt(total, out=self.grad_norm)
            if max_norm is not None and max_norm > 0:
                torch.clamp(max_norm / (self.grad_norm + 1e-6), max=1.0, out=self.grad_scale)
            else:
                self.grad_scale.fill_(1.0)
            return self.grad_norm
        self._sq3.zero_()
        for g in self.groups:
            lo, hi = g.shard_range
            if g.ep_sharded:
                self._sumsq_into(g.grad[lo:hi], 2)
                continue
            cut = min(max(g.n_tp_sharded, lo), hi)
            self._sumsq_into(g.grad[lo:cut], 1)
            self._sumsq_into(g.grad[cut:hi], 0)
        if self.world > 1:
            dist.all_reduce(self._sq3, group=self.pg)
        tp = getattr(self.model, "tp", None)
        if tp is not None:
            dist.all_reduce(self._sq3[1:2], group=tp.group)
        ep_group = getattr(self.model, "ep_group", None)
        if ep_group is not None and not getattr(self.model, "ep_in_dp", False):
            dist.all_reduce(self._sq3[2:3], group=ep_group)
        total = self._sq3.sum().reshape(1)
        for grp in extra_groups:
            dist.all_reduce(total, group=grp)
        torch.sqrt(total, out=self.grad_norm)
        if max_norm is not None and max_norm > 0:
            torch.clamp(max_norm / (self.grad_norm + 1e-6), max=1.0, out=self.grad_scale)
        else:
            self.grad_scale.fill_(1.0)
        return self.grad_norm

    # ------------------------------------------------------------------ hand-written training loops
    def bind_optimizer(self, optimizer) -> None:
        """Make ``loss.backward(); clip_grad_norm_(model, c); optimizer.step(); optimizer.zero_grad()`` a complete
        training step, as it is with FSDP2 in the reference: the step folds / reduces the gradients first when
        :meth:`finish_backward` has not run since the last ``zero_grad``, applies a pending clip factor, publishes the
        update afterwards, and ``optimizer.zero_grad`` also resets the flat gradient buffers.  A loop that drives the
        engine itself (``finish_backward`` ... ``after_optimizer_step``, as the trainer does) is not affected: the
        hooks find nothing left to do."""
        if getattr(optimizer, "_kf_engine_bound", None) is self:
            return
        fused = bool(getattr(optimizer, "_flat_groups", None))
        if fused:
            optimizer.grad_scale = self.grad_scale
        else:
            self.full_grads = True    # it steps on whole parameters: every rank needs the whole averaged gradient

        def before(_opt, _args, _kwargs):
            if not self._reduced:
                self.finish_backward()
                self._manual_step = True
            if self._manual_step and self._scale_pending and not fused:
                self.apply_grad_scale()

        def after(_opt, _args, _kwargs):
            if self._manual_step:
                self._manual_step = False
                self.after_optimizer_step()
                self._scale_pending = False    # a clip factor belongs to the step it was computed for
                self.grad_scale.fill_(1.0)

        optimizer.register_step_pre_hook(before)
        optimizer.register_step_post_hook(after)
        plain_zero_grad = optimizer.zero_grad

        def zero_grad(set_to_none: bool = True):
            plain_zero_grad(set_to_none=set_to_none)
            self.zero_grad()

        optimizer.zero_grad = zero_grad
        optimizer._kf_engine_bound = self

    def apply_grad_scale(self) -> None:
        """Multiply the (shard) gradients by ``grad_scale``; only needed for optimizers that do not fuse it."""
        self._scale_pending = False
        for g in self.groups:
            lo, hi = (0, g.numel) if self.full_grads else g.shard_range
            g.grad[lo:hi].mul_(self.grad_scale.to(g.grad.dtype))

    def publish_on_side_stream(self, flat_groups) -> bool:
        """True when the optimizer should hand its fused update + publication kernels to
        :meth:`publish_in_forward_order` (symmetric transport on a GPU, every unit in a symmetric buffer)."""
        if self._comm_stream is None or not self._handles:
            return False
        same = len(flat_groups) == len(self.groups) and all(a is b for a, b in zip(flat_groups, self.groups))
        if self.overlap_update:
            return same and all(g.param.numel() > 0 for g in self.groups)
        if not self.symmetric or os.environ.get("KF_DP_OVERLAP_PUBLISH", "1") == "0":
            return False
        return same and all(getattr(g, "param_symm", None) is not None and g.param.numel() > 0 for g in self.groups)

    def publish_in_forward_order(self, launch) -> None:
        """Run ``launch(unit)`` (sharded optimizer update that stores the new parameters on every rank) for every
        unit on the communication stream: root unit first (the embedding is needed first), then the blocks in
        order.  Each launch is followed by that unit's cross-rank barrier (all ranks' stores into this rank's copy
        are complete) and an event; a unit's next forward waits for its own event (``wait_params``), so the update
        of the later blocks overlaps the forward pass of the earlier ones."""
        order = list(self._root_groups) + [i for i in range(len(self.groups)) if i not in set(self._root_groups)]
        ready = torch.cuda.Event()
        ready.record()  # gradients reduced, clipping scale and skip flag final
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ready)
            for i in order:
                g = self.groups[i]
                launch(g)
                if self.world > 1:
                    g.param_symm.barrier()
                done = torch.cuda.Event()
                done.record()
                self._gather_work[i] = _EventWork(done)
        self._published_per_group = True

    def after_optimizer_step(self) -> None:
        """Publish the updated shards so that every rank holds the full new parameters.  On GPUs the
        all-gathers are asynchronous and each block waits for its own only when its next forward starts."""
        if self._published_per_group:
            self._published_per_group = False  # every unit carries its own (barrier +) event
            return
        if self.symmetric:
            # the optimizer kernel already stored the new parameters on every rank; one barrier makes sure all
            # ranks' stores (and their reads of our gradients) are complete before the next step touches them
            self.groups[-1].param_symm.barrier()
            return
        if self.world > 1:
            use_async = self.groups[0].param.is_cuda and bool(self._group_of_module is not None)
            for i, g in enumerate(self.groups):
                if g.local:
                    continue
                lo, hi = g.shard_range
                if use_async:
                    self._gather_work[i] = dist.all_gather_into_tensor(g.param, g.param[lo:hi], group=self.pg, async_op=True)
                else:
                    dist.all_gather_into_tensor(g.param, g.param[lo:hi].clone(), group=self.pg)

    def release(self) -> None:
        """Detach from the model (before another engine is built over a changed set of trainable parameters):
        drains communication, removes hooks and wrappers, and gives every parameter storage of its own."""
        self.wait_all()
        for h in self._handles + getattr(self, "_aux_handles", []):
            h.remove()
        self._handles.clear()
        self._aux_handles = []
        for name in self._wrapped:
            self.model.__dict__.pop(name, None)
        self._wrapped.clear()
        for g in self.groups:
            for p in g.params:
                p.data = p.data.clone()
                p.grad = None
                for attr in ("_kf_grad", "_kf_grad_live"):
                    if hasattr(p, attr):
                        delattr(p, attr)
        self.groups = []
        if getattr(self.model, "_kf_engine", None) is self:
            del self.model._kf_engine

    def wait_all(self) -> None:
        """Drain every in-flight reduction / publication (before checkpoints, evaluation, shutdown)."""
        for table in (self._reduce_work, self._gather_work):
            for i in list(table):
                table.pop(i).wait()

    def zero_grad(self) -> None:
        for g in self.groups:
            g.zero_grad()
            g._kf_ep_scaled = False
            for p in g.params:
                if getattr(p, "_kf_tp_synced", False):
                    p._kf_tp_synced = False
        self._reduced = False
        self._expose_queued = False

    # ------------------------------------------------------------------ checkpoint helpers
    def full_optimizer_state(self, g: FlatParamGroup) -> tuple[torch.Tensor, torch.Tensor]:
        """Whole-unit moment buffers assembled from every rank's shard."""
        if self.world == 1 or g.local:
            return g.exp_avg, g.exp_avg_sq
        out = []
        for shard in (g.exp_avg, g.exp_avg_sq):
            full = torch.empty(g.numel, dtype=shard.dtype, device=shard.device)
            dist.all_gather_into_tensor(full, shard, group=self.pg)
            out.append(full)
        return out[0], out[1]

    def load_full_optimizer_state(self, g: FlatParamGroup, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor) -> None:
        lo, hi = g.shard_range
        g.exp_avg.copy_(exp_avg[lo:hi])
        g.exp_avg_sq.copy_(exp_avg_sq[lo:hi])


class _EventWork:
    """Handle of work queued on the communication stream: ``wait`` makes the current stream wait for it."""

    def __init__(self, event) -> None:
        self.event = event

    def wait(self) -> None:
        torch.cuda.current_stream().wait_event(self.event)


class _CopyAfterWork:
    """Handle of an asynchronous reduction into a wide buffer whose result is then rounded into the gradient shard."""

    def __init__(self, work, src: torch.Tensor, dst: torch.Tensor, keep) -> None:
        self.work, self.src, self.dst, self.keep = work, src, dst, keep

    def wait(self) -> None:
        self.work.wait()
        self.dst.copy_(self.src)
        self.keep = None


class _ScaledWork:
    """Handle of an asynchronous sum whose result still has to be divided by the world size."""

    def __init__(self, work, tensor: torch.Tensor, world: int) -> None:
        self.work, self.tensor, self.world = work, tensor, world

    def wait(self) -> None:
        self.work.wait()
        self.tensor.div_(self.world)


def clip_grad_norm_(model: nn.Module, max_norm: float, foreach: bool | None = None) -> torch.Tensor:
    """Clip the global gradient norm in place; returns the pre-clip norm.  Engine-aware."""
    engine = getattr(model, "_kf_engine", None)
    if engine is not None:
        if not engine._reduced:            # a hand-written loop: nobody has reduced this step's gradients yet
            engine.finish_backward()
            engine._manual_step = True
        norm = engine.clip_grad_norm(max_norm)
        engine._scale_pending = True
        return norm.reshape(())
    grads = [p.grad for p in model.parameters() if p.grad is not None]
    if not grads:
        return torch.zeros(())
    local = [g.to_local() if hasattr(g, "to_local") else g for g in grads]
    total = torch.sqrt(sum(g.float().pow(2).sum() for g in local))
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for g in local:
        g.mul_(coef.to(g.dtype))
    return total
