"""Pipeline parallelism: contiguous layer ranges per stage and our own GPipe / 1F1B schedules.

Stage 0 owns the token embedding, the last stage owns the final norm and the output head; layers are
split evenly with the remainder going to the early stages; layer keys stay global so checkpoint names do
not depend on the split.  Activations and their gradients cross stage boundaries with point-to-point
``torch.distributed`` operations (NCCL on GPUs, gloo on CPU); sends and receives of one schedule slot are
posted together (``batch_isend_irecv``) so neighbouring stages can never dead-lock on ordering, and on
GPUs they run asynchronously to the compute stream.  Parameters stay resident (no re-sharding between
micro-batches).  The mean loss and the gradient norm are shared from the last stage over the pipeline group.

Parity: kempnerforge/distributed/pipeline_parallel.py:77-365 and the pipeline step of
scripts/train.py:684-740 (n_microbatches = grad_accum_steps, schedules ``1f1b`` and ``gpipe``;
``interleaved_1f1b`` needs several stages per rank and is rejected like in the reference's wiring).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from kempnerforge_b200.models.modality import ModalityContext
from kempnerforge_b200.models.transformer import Transformer
from kempnerforge_b200.parallel.setup import mesh_dim


def compute_layer_assignment(n_layers: int, pp_size: int) -> list[tuple[int, int]]:
    """``(start, end)`` layer range of every stage, end exclusive: an even split in which the first
    ``n_layers % pp_size`` stages get one more.  Parity: kempnerforge/distributed/pipeline_parallel.py:77-112."""
    if pp_size <= 0:
        raise ValueError("pp_size must be positive")
    if n_layers < pp_size:
        raise ValueError(f"pp_size ({pp_size}) cannot exceed n_layers ({n_layers})")
    base, extra = divmod(n_layers, pp_size)
    out, start = [], 0
    for s in range(pp_size):
        n = base + (1 if s < extra else 0)
        out.append((start, start + n))
        start += n
    return out


class PipelineStageModule(Transformer):
    """The slice of the transformer owned by one pipeline stage."""

    def __init__(self, config, pp_rank: int | None = None, pp_size: int | None = None,
                 layer_range: tuple[int, int] | None = None, *, stage_id: int | None = None,
                 num_stages: int | None = None) -> None:
        """Stage ``pp_rank`` of ``pp_size`` (also spelled ``stage_id`` / ``num_stages``); ``layer_range = (start, end)``
        overrides the balanced layer assignment."""
        pp_rank = stage_id if pp_rank is None else pp_rank
        pp_size = num_stages if pp_size is None else pp_size
        if pp_rank is None or pp_size is None:
            raise TypeError("PipelineStageModule needs the stage index and the number of stages")
        layers = list(range(*(layer_range if layer_range is not None
                              else compute_layer_assignment(config.n_layers, pp_size)[pp_rank])))
        super().__init__(config, layer_ids=layers, with_embedding=pp_rank == 0, with_head=pp_rank == pp_size - 1)
        self.pp_rank, self.pp_size = pp_rank, pp_size
        self.is_first, self.is_last = pp_rank == 0, pp_rank == pp_size - 1

    def forward(self, x: torch.Tensor, doc_ids=None) -> torch.Tensor:  # type: ignore[override]
        """tokens (first stage) or hidden states -> hidden states (the last stage applies the final norm)."""
        if self.is_first:
            return self.forward_hidden(x, doc_ids=doc_ids)
        return self.forward_hidden(None, modality=ModalityContext(inputs_embeds=x), doc_ids=doc_ids)

    def init_weights_and_freqs(self) -> None:
        """(Re-)draw this stage's weights and build its rotary tables, e.g. after ``to_empty`` on a meta build."""
        from kempnerforge_b200.models.init import init_weights

        device = next(self.parameters()).device
        init_weights(self, self.config)
        self._rope_cos = None
        self.rope_tables(device, 0, 1)

    def stage_loss(self, hidden: torch.Tensor, labels: torch.Tensor, z_loss_weight: float = 0.0) -> torch.Tensor:
        from kempnerforge_b200.ops import functional as F

        return F.linear_cross_entropy(hidden, self.output_head.proj.weight, labels, z_loss_weight)


def build_stage_module(config, pp_rank: int, pp_size: int) -> PipelineStageModule:
    return PipelineStageModule(config, pp_rank, pp_size)


def build_pipeline_stage(stage_module: PipelineStageModule, device_mesh, device: torch.device, batch_size: int = 0,
                         seq_len: int = 0, param_dtype: torch.dtype = torch.bfloat16, schedule: str = "1f1b"):
    """A runnable stage (``PipelineRunner``) for a stage module: moves it to ``device`` / ``param_dtype`` and binds the
    pipeline process group of ``device_mesh``.  Activation shapes are taken from the first micro-batch, so
    ``batch_size`` and ``seq_len`` are accepted only for call compatibility.
    Parity: kempnerforge/distributed/pipeline_parallel.py:259-306."""
    pp_mesh = get_pp_mesh(device_mesh)
    stage_module.to(device=device, dtype=param_dtype)
    stage_module.rope_tables(device, 0, 1)
    return PipelineRunner(stage_module, pp_mesh.get_group() if pp_mesh is not None else None, schedule)


def get_pp_mesh(device_mesh):
    return device_mesh["pp"] if device_mesh is not None and "pp" in (device_mesh.mesh_dim_names or ()) else None


_STAGE_GROUPS: dict[int, object] = {}


def stage_process_group(mesh):
    """The process group of all ranks that hold the same pipeline stage as this rank (its data- / tensor-parallel
    peers); checkpoints of a stage are coordinated inside it.  Every rank creates every stage's group, in stage
    order, the first time this is called for a mesh."""
    import torch.distributed as dist

    names = tuple(mesh.mesh_dim_names or ())
    if "pp" not in names:
        return None
    key = id(mesh)
    if key not in _STAGE_GROUPS:
        grid = mesh.mesh.movedim(names.index("pp"), 0)
        mine = None
        for stage in range(grid.shape[0]):
            ranks = sorted(int(r) for r in grid[stage].flatten().tolist())
            group = dist.new_group(ranks)
            if dist.get_rank() in ranks:
                mine = group
        _STAGE_GROUPS[key] = mine
    return _STAGE_GROUPS[key]


def get_pp_rank(device_mesh) -> int:
    return mesh_dim(device_mesh, "pp")[2]


def get_pp_size(device_mesh) -> int:
    return mesh_dim(device_mesh, "pp")[1]


# --------------------------------------------------------------------------- schedules
def schedule_order(kind: str, stage: int, n_stages: int, n_micro: int) -> list[tuple[str, int]]:
    """The sequence of ("F", i) / ("B", i) slots one stage executes."""
    kind = str(kind)
    if kind == "gpipe":
        return [("F", i) for i in range(n_micro)] + [("B", i) for i in range(n_micro)]
    if kind != "1f1b":
        raise ValueError(f"unsupported pipeline schedule {kind!r} (interleaved schedules need several stages per rank)")
    warm = min(n_stages - stage - 1, n_micro)
    order = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < n_micro:
        order.append(("F", f))
        order.append(("B", b))
        f, b = f + 1, b + 1
    while b < n_micro:
        order.append(("B", b))
        b += 1
    return order


class PipelineRunner:
    def __init__(self, module: PipelineStageModule, pp_group, schedule: str = "1f1b") -> None:
        self.module = module
        self.group = pp_group
        self.size = dist.get_world_size(pp_group)
        self.rank = dist.get_rank(pp_group)
        self.schedule = str(schedule)
        self.prev = dist.get_global_rank(pp_group, self.rank - 1) if self.rank > 0 else None
        self.next = dist.get_global_rank(pp_group, self.rank + 1) if self.rank < self.size - 1 else None
        self.last_global = dist.get_global_rank(pp_group, self.size - 1)
        p = next(module.parameters())
        self.dtype, self.device = p.dtype, p.device

    # -- point to point -------------------------------------------------------
    def _exchange(self, sends: list[tuple[torch.Tensor, int]], recvs: list[tuple[torch.Tensor, int]]) -> None:
        ops = [dist.P2POp(dist.isend, t.contiguous(), peer, group=self.group) for t, peer in sends]
        ops += [dist.P2POp(dist.irecv, t, peer, group=self.group) for t, peer in recvs]
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def run_step(self, micro_batches: list[dict], z_loss_weight: float = 0.0) -> torch.Tensor:
        """Forward + backward of all micro-batches; returns the mean loss (valid on the last stage, else 0).

        Communication follows the classic non-interleaved pattern: in the steady state a stage posts
        "send activation forward + receive gradient" as one batch and "send gradient backward + receive next
        activation" as another, so a pair of neighbours never waits on each other in opposite directions.
        """
        m = self.module
        n = len(micro_batches)
        mb, s = micro_batches[0]["input_ids"].shape
        shape = (mb, s, m.config.dim)
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        m.train()
        new_buf = lambda: torch.empty(shape, dtype=self.dtype, device=self.device)  # noqa: E731
        inputs: dict[int, torch.Tensor | None] = {}
        outputs: dict[int, torch.Tensor] = {}

        def recv_forward():
            if m.is_first:
                return None
            x = new_buf()
            self._exchange([], [(x, self.prev)])
            return x

        def forward(i: int, x):
            nonlocal total
            batch = micro_batches[i]
            if m.is_first:
                x = batch["input_ids"]
            else:
                x.requires_grad_(True)
            inputs[i] = x
            h = m(x, doc_ids=batch.get("doc_ids"))
            if m.is_last:
                h = m.stage_loss(h, batch["labels"], z_loss_weight) / n
                total += h.detach().float()
            outputs[i] = h
            return h

        def backward(i: int, grad):
            out = outputs.pop(i)
            if m.is_last:
                out.backward()
            else:
                out.backward(grad)
            x = inputs.pop(i)
            return None if m.is_first else x.grad

        if self.schedule == "gpipe":
            warm = n
        elif self.schedule == "1f1b":
            warm = min(self.size - self.rank - 1, n)
        else:
            raise ValueError(f"unsupported pipeline schedule {self.schedule!r}")
        steady = n - warm
        f = b = 0
        for _ in range(warm):  # warm-up forwards
            h = forward(f, recv_forward())
            if not m.is_last:
                self._exchange([(h.detach(), self.next)], [])
            f += 1
        x = recv_forward() if steady > 0 else None
        for j in range(steady):  # one forward, one backward
            h = forward(f, x)
            f += 1
            grad = None
            if not m.is_last:
                grad = new_buf()
                self._exchange([(h.detach(), self.next)], [(grad, self.next)])
            gin = backward(b, grad)
            b += 1
            last = j == steady - 1
            if m.is_first:
                x = None
            elif last:
                self._exchange([(gin, self.prev)], [])
            else:
                x = new_buf()
                self._exchange([(gin, self.prev)], [(x, self.prev)])
        for _ in range(warm):  # cool-down backwards
            grad = None
            if not m.is_last:
                grad = new_buf()
                self._exchange([], [(grad, self.next)])
            gin = backward(b, grad)
            b += 1
            if not m.is_first:
                self._exchange([(gin, self.prev)], [])
        return total

    @torch.no_grad()
    def eval_loss(self, input_ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        m = self.module
        shape = (*input_ids.shape, m.config.dim)
        if m.is_first:
            x = input_ids
        else:
            x = torch.empty(shape, dtype=self.dtype, device=self.device)
            self._exchange([], [(x, self.prev)])
        h = m(x)
        loss = torch.zeros((), dtype=torch.float32, device=self.device)
        if m.is_last:
            loss = m.stage_loss(h, labels).float()
        else:
            self._exchange([(h, self.next)], [])
        dist.broadcast(loss, src=self.last_global, group=self.group)
        return loss

    def clip_grad_norm(self, model, max_norm: float) -> torch.Tensor:
        engine = getattr(model, "_kf_engine", None)
        return engine.clip_grad_norm(max_norm, extra_groups=(self.group,)).reshape(())

    def share_scalars(self, vec: torch.Tensor) -> None:
        """Overwrite ``vec`` on every stage with the last stage's values (loss; the norm is already global)."""
        keep = vec[1].clone()
        dist.broadcast(vec, src=self.last_global, group=self.group)
        vec[1] = keep


def build_pipeline(config, device: torch.device, mesh, transport: str | None = None) -> PipelineRunner:
    """Stage module -> (TP) -> (fp8) -> AC -> sharded DP, plus the schedule runner."""
    from kempnerforge_b200.parallel.parallel import apply_ac, apply_float8, apply_fsdp2

    group, size, rank = mesh_dim(mesh, "pp")
    tc = config.train
    with torch.device(device):
        module = build_stage_module(config.model, rank, size)
    module = module.to(device=device, dtype=tc.param_dtype)
    if mesh_dim(mesh, "tp")[1] > 1:
        from kempnerforge_b200.parallel.tensor_parallel import apply_tensor_parallel

        apply_tensor_parallel(module, mesh)
    if tc.is_fp8:
        apply_float8(module)
    if str(tc.activation_checkpointing) != "none":
        apply_ac(module, str(tc.activation_checkpointing))
    apply_fsdp2(module, mesh, transport=transport)
    return PipelineRunner(module, group, str(config.distributed.pp_schedule))


def build_pipeline_schedule(runner: PipelineRunner, n_microbatches: int, loss_fn=None,
                            schedule: str = "1f1b") -> list[tuple[str, int]]:
    """The slot list this rank will execute (exposed for inspection and tests).  ``loss_fn`` is accepted for call
    compatibility (the last stage computes its loss with the fused head + cross-entropy); a schedule name in its
    place is understood too."""
    if isinstance(loss_fn, str):
        schedule = loss_fn
    return schedule_order(schedule, runner.rank, runner.size, n_microbatches)
