"""Sharded-parameter data parallelism (ZeRO-3) over flat units.

Memory plan: for every transformer block each rank keeps piece ``rank`` of every parameter (``FlatParamGroup``
with ``sharded=True``), the matching gradient shard and the moments — 1/N of everything.  Whole parameters and
whole gradients exist only in *staging* buffers shared by all blocks: one parameter staging buffer (the size of
the largest block) and two gradient staging buffers (block i reduces while block i-1 computes).  The root unit
(embedding, final norm, head) stays in the resident scheme of :class:`DataParallelEngine`.

Forward of a block: nothing is gathered ahead of time.  Each GEMM of the fused dense block pulls ITS weight rows
from the peers' shards inside the GEMM kernel (``kf_gemm_gather_bf16``: copy warps issue NVLink peer loads into
the staging buffer, the TMA producer follows their progress through per-row-block counters), so the all-gather is
overlapped with the very GEMM that consumes it.  The few non-matrix parameters are pulled by a small kernel
(``kf_symm_pull_bf16``).  Backward of a block: the recomputation gathers again the same way (reshard-after-forward
semantics); weight gradients are written into a gradient staging buffer and reduce-scattered into the gradient
shard by ``kf_symm_rs_shard_bf16`` on the communication stream, overlapping the previous block's backward.

The kernels never wait for another GPU.  Ordering between ranks is: one barrier after the optimizer step (every
shard is final before anybody pulls it) and, per block, one barrier before the gradient reduction (all ranks
wrote their gradients) and one after it (all ranks finished reading this rank's staging buffer).

Off GPUs (gloo) and with ``transport="collective"`` the same engine runs on ``all_gather`` / ``all_reduce``.

Replaces ``fully_shard(..., reshard_after_forward=True)`` of the reference
(kempnerforge/distributed/parallel.py:184-302).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from kempnerforge_b200.parallel.engine import DataParallelEngine, _EventWork
from kempnerforge_b200.parallel.flat import FlatParamGroup

GATHER_CHUNK = 16384  # elements moved per copy step of the gathering GEMM (pieces must be multiples of it)


class ShardedDataParallelEngine(DataParallelEngine):
    shard_blocks = True

    def __init__(self, model: nn.Module, process_group=None, transport: str = "collective", allocator=None) -> None:
        if process_group is not None and dist.get_world_size(process_group) > 1:
            # every rank starts from rank 0's weights: broadcast BEFORE the parameters are cut into pieces
            root = dist.get_global_rank(process_group, 0)
            seen = set()
            for p in model.parameters():
                if id(p) not in seen and p.requires_grad:
                    seen.add(id(p))
                    dist.broadcast(p.data, src=root, group=process_group)
        super().__init__(model, process_group, transport=transport, allocator=allocator)
        self.sharded_groups: list[FlatParamGroup] = [g for g in self.groups if g.sharded]
        self._stage_owner: FlatParamGroup | None = None
        self._grad_slot_free: list = [None, None]
        self.shared_staging = False
        self.use_kernels = False
        if not self.sharded_groups:
            return
        dev, dt = self.device, self.sharded_groups[0].dtype
        # On a GPU all blocks share the staging buffers (this is where the memory is saved; it needs the fused dense
        # block, which writes every gradient into the staging buffer and re-gathers in its own backward).  Elsewhere
        # (CPU tests of the plumbing) every unit gets staging of its own and the ordinary autograd path works.
        self.shared_staging = dev.type == "cuda"
        if not self.shared_staging:
            self.use_kernels = False
            self._gather_flags = None
            for g in self.sharded_groups:
                g.engine = self
                g.slot = 0
                g.bind(torch.zeros(g.numel, dtype=dt, device=dev), torch.zeros(g.numel, dtype=dt, device=dev), None)
                self.pull(g, list(range(len(g.params))))
                g.valid = {"all"}
            return
        n_max = max(g.numel for g in self.sharded_groups)
        self.param_stage = torch.empty(n_max, dtype=dt, device=dev)
        alloc = allocator or (lambda n, d, dv: torch.zeros(n, dtype=d, device=dv))
        self.grad_stages = [alloc(n_max, dt, dev) for _ in range(2)]
        self._grad_stage_symm = [None, None]
        if allocator is not None:
            from kempnerforge_b200.comm import symmetric

            self._grad_stage_symm = [symmetric.lookup(t) for t in self.grad_stages]
        self.use_kernels = bool(self.symmetric or (allocator is not None and self.world > 1)) and dev.type == "cuda"
        if self.use_kernels and self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream()
        self._gather_flags = torch.zeros(8192, dtype=torch.int32, device=dev) if dev.type == "cuda" else None
        for k, g in enumerate(self.sharded_groups):
            g.engine = self
            g.slot = k % 2
            g.bind(self.param_stage, self.grad_stages[g.slot], self._grad_stage_symm[g.slot])
        if self.use_kernels:
            self.sharded_groups[0].shard_symm.barrier()

    # ------------------------------------------------------------------ set-up
    def broadcast_parameters(self, src: int = 0) -> None:
        root = dist.get_global_rank(self.pg, src) if self.pg is not None else src
        for g in self.groups:
            if g.local or g.sharded:
                continue
            dist.broadcast(g.param, src=root, group=self.pg)

    def _make_pre_hook(self, idxs):
        def hook(module, args):
            self.wait_params(idxs)
            for i in idxs:
                g = self.groups[i]
                if g.sharded:
                    self.acquire(g, everything=not torch.is_grad_enabled())
            x = args[0] if args else None
            if torch.is_tensor(x) and x.requires_grad and torch.is_grad_enabled():
                x.register_hook(lambda grad, idxs=idxs: self._block_backward_done(idxs))

        return hook

    # ------------------------------------------------------------------ parameter staging
    def acquire(self, g: FlatParamGroup, everything: bool = False) -> None:
        """Make ``g`` the owner of the parameter staging buffer.  Matrices are gathered later by the GEMMs that read
        them (or by :meth:`ensure`); the remaining small parameters are pulled here.  ``everything``: pull the whole
        unit now (evaluation, generation and any code path outside the fused block)."""
        if self.shared_staging and self._stage_owner is not g:
            self._stage_owner = g
            g.valid = set()
        if everything or not self.shared_staging:
            if "all" not in g.valid:
                self.pull(g, list(range(len(g.params))))
                g.valid = {"all"}
            return
        if "small" not in g.valid and "all" not in g.valid:
            small = [i for i, p in enumerate(g.params) if p.dim() < 2]
            if small:
                self.pull(g, small)
            g.valid.add("small")

    def ensure(self, g: FlatParamGroup, key: str, weights) -> None:
        """The parameters ``weights`` of ``g`` hold their current values in the staging buffer (pulls them if not)."""
        if not self.shared_staging or self._stage_owner is not g:
            self.acquire(g)
        if key in g.valid or "all" in g.valid:
            return
        self.pull(g, [g.index_of(w) for w in weights])
        g.valid.add(key)

    def pull(self, g: FlatParamGroup, idxs: list[int]) -> None:
        """All-gather the listed parameters of ``g`` into the parameter staging buffer."""
        if not idxs:
            return
        w = self.world
        if self.use_kernels:
            from kempnerforge_b200.ops import cuda as kcuda

            for lo in range(0, len(idxs), 16):
                part = idxs[lo : lo + 16]
                kcuda.symm_pull(g.shard_symm, [g.offsets[i] for i in part], [g.padded[i] for i in part],
                                [g.offsets[i] // w for i in part], g.param)
            return
        gathered = torch.empty(w * g.shard_numel, dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(gathered, g.shard, group=self.pg)
        rows = gathered.view(w, g.shard_numel)
        for i in idxs:
            o, n = g.offsets[i], g.padded[i]
            g.param[o : o + n].view(w, n // w).copy_(rows[:, o // w : (o + n) // w])

    def gather_plan(self, g: FlatParamGroup, weights, k: int):
        """Arguments for the weight-gathering GEMM over the row stack ``weights`` (all of ``g``), or None when the
        shapes do not fit its granularity (the caller then pulls with :meth:`ensure` and runs the plain GEMM)."""
        if not self.use_kernels or k % 128:
            return None
        idx = [g.index_of(w_) for w_ in weights]
        for a, b in zip(idx, idx[1:]):
            if g.offsets[a] + g.padded[a] != g.offsets[b]:
                return None
        for i, w_ in zip(idx, weights):
            if g.padded[i] != w_.numel() or w_.dim() != 2 or w_.shape[1] != k or (w_.numel() // self.world) % GATHER_CHUNK:
                return None
        rows = sum(w_.shape[0] for w_ in weights)
        if rows % 128 or rows // 128 + 1 > self._gather_flags.numel():
            return None
        stage = g.param[g.offsets[idx[0]] : g.offsets[idx[0]] + rows * k]
        return {"symm": g.shard_symm, "seg_rows": [w_.shape[0] for w_ in weights],
                "seg_src": [g.offsets[i] // self.world for i in idx], "stage": stage, "flags": self._gather_flags}

    # ------------------------------------------------------------------ gradients
    def prepare_backward(self, g: FlatParamGroup) -> None:
        """Called when a block's backward starts: the block owns the parameter staging again (its matrices are
        gathered once more by the recomputation) and its gradient staging buffer must have been released by the
        reduction that used it last."""
        self.acquire(g)
        ev = self._grad_slot_free[g.slot]
        if ev is not None:
            ev.wait()
            self._grad_slot_free[g.slot] = None

    def _block_backward_done(self, idxs) -> None:
        if self.world <= 1 or not self.shared_staging:
            return None   # separate staging per unit: gradients are folded and reduced in finish_backward
        for i in idxs:
            g = self.groups[i]
            if not g.sharded:
                continue
            if not all(getattr(p, "_kf_grad_live", False) for p in g.params):
                raise RuntimeError(
                    f"unit {g.name}: sharded parameters need the fused dense block (every gradient is written into the "
                    "gradient staging buffer); this block ran on a path that does not do that")
            work = self._reduce_sharded(g)
            self._grad_slot_free[g.slot] = work
            self._reduce_work[i] = work
            for p in g.params:
                p._kf_grad_live = False
        return None

    def _reduce_sharded(self, g: FlatParamGroup):
        """grad_shard (+)= mean over ranks of the pieces of this rank inside every rank's gradient staging buffer."""
        w = self.world
        accumulate = g.grad_shard_live
        g.grad_shard_live = True
        if self.use_kernels:
            from kempnerforge_b200.ops import cuda as kcuda

            symm = g.grad_stage_symm
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ready)
                symm.barrier()   # every rank has written this block's gradients
                for lo in range(0, len(g.params), 16):
                    part = list(range(lo, min(lo + 16, len(g.params))))
                    kcuda.symm_rs_shard(symm, [g.offsets[i] for i in part], [g.padded[i] for i in part],
                                        [g.offsets[i] // w for i in part], g.grad_shard, accumulate)
                symm.barrier()   # every rank has finished reading this rank's staging buffer
                done = torch.cuda.Event()
                done.record()
            return _EventWork(done)
        tmp = torch.empty(w, g.shard_numel, dtype=g.dtype, device=g.device)
        for o, n in zip(g.offsets, g.padded):
            tmp[:, o // w : (o + n) // w].copy_(g.grad[o : o + n].view(w, n // w))
        if g.grad.is_cuda and "nccl" in str(dist.get_backend(self.pg)):
            out = torch.empty(g.shard_numel, dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, tmp.view(-1), op=dist.ReduceOp.AVG, group=self.pg)
        else:
            dist.all_reduce(tmp, group=self.pg)
            out = tmp[self.rank].div_(w)
        if accumulate:
            g.grad_shard.add_(out)
        else:
            g.grad_shard.copy_(out)
        return _DoneWork()

    def _reduce_gradients(self) -> None:
        for i, g in enumerate(self.groups):
            if g.sharded:
                work = self._reduce_work.pop(i, None)
                if work is not None:
                    work.wait()
                elif not self.shared_staging:
                    self._reduce_sharded(g)
                continue
            if g.local:
                g.grad.div_(self.world)
                continue
            work = self._reduce_work.pop(i, None)
            if work is not None:
                work.wait()
                continue
            self._reduce_one(g)

    def finish_backward(self) -> None:
        for g in self.groups:
            g.finalize_grads()   # a no-op for units on shared staging
        if self.world > 1 and (self.requires_sync or self.shared_staging):
            self._reduce_gradients()
        self._reduced = True

    def clip_grad_norm(self, max_norm: float | None, extra_groups=()) -> torch.Tensor:
        if not self._sq_from_reduce:
            self._sq3.zero_()
            for g in self.groups:
                if g.sharded:
                    continue
                lo, hi = g.shard_range
                self._sumsq_into(g.grad[lo:hi], 0)
        self._sq_from_reduce = False
        for g in self.sharded_groups:
            self._sumsq_into(g.grad_shard, 0)
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

    def apply_grad_scale(self) -> None:
        self._scale_pending = False
        for g in self.groups:
            if g.sharded:
                g.grad_shard.mul_(self.grad_scale.to(g.grad_shard.dtype))
            else:
                lo, hi = (0, g.numel) if self.full_grads else g.shard_range
                g.grad[lo:hi].mul_(self.grad_scale.to(g.grad.dtype))

    def publish_on_side_stream(self, flat_groups) -> bool:
        return False

    def after_optimizer_step(self) -> None:
        """The shards changed: whatever the staging buffer holds is stale, and no rank may pull before every rank
        has finished its update (one barrier; the root unit publishes as in the resident engine)."""
        self._stage_owner = None
        for g in self.sharded_groups:
            g.valid = set()
        if self.world <= 1:
            return
        if not self.shared_staging:
            for g in self.sharded_groups:   # the ordinary autograd path reads whole parameters at any time
                self.acquire(g, everything=True)
        if self.symmetric:
            self.groups[-1].param_symm.barrier() if self.groups[-1].param_symm is not None else \
                self.sharded_groups[0].shard_symm.barrier()
            return
        if self.use_kernels:
            self.sharded_groups[0].shard_symm.barrier()
        for g in self.groups:
            if g.local or g.sharded:
                continue
            lo, hi = g.shard_range
            dist.all_gather_into_tensor(g.param, g.param[lo:hi].clone(), group=self.pg)

    def release(self) -> None:
        raise RuntimeError("the sharded-parameter engine cannot be released and rebuilt (freeze schedules need the "
                           "resident engine)")

    # ------------------------------------------------------------------ whole tensors for checkpoints / tests
    def full_parameter(self, p) -> torch.Tensor:
        """The current whole value of a sharded parameter (a fresh tensor assembled from every rank's piece)."""
        g = p._kf_flat
        i = g.index_of(p)
        w, n = self.world, g.padded[i]
        out = torch.empty(n, dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.piece_of(p).contiguous(), group=self.pg)
        return out[: p.numel()].view(p.shape)

    def load_full_parameter(self, p, value: torch.Tensor) -> None:
        g = p._kf_flat
        i = g.index_of(p)
        piece = g.padded[i] // self.world
        flat = value.reshape(-1)
        lo, hi = self.rank * piece, min((self.rank + 1) * piece, flat.numel())
        dst = g.piece_of(p)
        dst.zero_()
        if hi > lo:
            dst[: hi - lo].copy_(flat[lo:hi])
        self._stage_owner = None
        g.valid = set()

    def memory_report(self) -> dict[str, float]:
        """GB held by this engine on this rank, by kind."""
        gb = 1.0 / (1 << 30)
        b = lambda t: 0 if t is None else t.numel() * t.element_size()  # noqa: E731
        if not getattr(self, "shared_staging", False):
            return {}
        rep = {"param_shards": sum(b(g.shard) for g in self.sharded_groups) * gb,
               "grad_shards": sum(b(g.grad_shard) for g in self.sharded_groups) * gb,
               "moments": sum(b(g.exp_avg) + b(g.exp_avg_sq) for g in self.groups) * gb,
               "staging": (b(getattr(self, "param_stage", None)) + sum(b(t) for t in getattr(self, "grad_stages", []))) * gb,
               "resident_units": sum(b(g.param) + b(g.grad) for g in self.groups if not g.sharded) * gb}
        rep["total"] = sum(rep.values())
        return rep


class _DoneWork:
    def wait(self) -> None:
        return None
