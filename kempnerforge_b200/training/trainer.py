"""The training loop as a library object.

``Trainer(config).fit()`` is what ``scripts/train.py`` runs; ``Trainer.train_step(batches)`` is the
unit a benchmark or a notebook can call directly.  A step is:

  for each micro-batch:  loss = CE(+z) + aux terms;  (loss / accum).backward()
  finish_backward()      fold / reduce gradients across data-parallel ranks
  clip                   global-norm clipping factor computed on the device
  NaN check              one host read per step (loss + grad norm + finite flag together)
  optimizer.step(); scheduler.step(); phase LR scale; zero_grad

The host reads exactly one small tensor per optimizer step (loss, gradient norm); per-micro-batch
losses are accumulated on the device.

Parity: scripts/train.py:69-1081 of the reference (same order of construction, resume, phase
schedule, hooks, MoE metrics, NCCL health checks, evaluation, checkpoint cadence, emergency and
final checkpoints, log strings ``Starting training: step=``, ``Training complete: N steps, T tokens``,
``Shutdown requested at step N``).
"""

from __future__ import annotations

from collections.abc import Iterator
from typing import Any

import torch
import torch.distributed as dist

from kempnerforge_b200.config.job import JobConfig
from kempnerforge_b200.metrics.logger import get_logger
from kempnerforge_b200.metrics.tracker import MetricsTracker
from kempnerforge_b200.parallel.engine import clip_grad_norm_
from kempnerforge_b200.parallel.parallel import build_parallel_model
from kempnerforge_b200.parallel.setup import get_dp_info, get_world_info, init_distributed, mesh_dim
from kempnerforge_b200.training.grad import maybe_no_sync
from kempnerforge_b200.training.hooks import HookRunner, StepContext, load_hooks
from kempnerforge_b200.training.optimizer import FusedAdamW, build_optimizer
from kempnerforge_b200.training.scheduler import build_scheduler

log = get_logger("trainer")


def _to_device(batch: dict[str, Any], device: torch.device) -> dict[str, Any]:
    return {k: (v.to(device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in batch.items()}


class SyntheticTokens:
    """Endless uniform-random token batches; labels are the inputs shifted by one.

    The generator is seeded with (seed, dp_rank) so data-parallel ranks see different data and a
    resumed run continues the same stream (its state is part of the checkpoint).
    """

    def __init__(self, vocab_size: int, batch_size: int, seq_len: int, seed: int, dp_rank: int = 0,
                 pin_memory: bool = False) -> None:
        self.vocab_size, self.batch_size, self.seq_len = vocab_size, batch_size, seq_len
        self.gen = torch.Generator().manual_seed(seed * 1000003 + dp_rank)
        self.pin = pin_memory and torch.cuda.is_available()
        self.batches_yielded = 0

    def __iter__(self) -> Iterator[dict[str, torch.Tensor]]:
        return self

    def __next__(self) -> dict[str, torch.Tensor]:
        tok = torch.randint(0, self.vocab_size, (self.batch_size, self.seq_len + 1), generator=self.gen)
        self.batches_yielded += 1
        ids, labels = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        if self.pin:
            ids, labels = ids.pin_memory(), labels.pin_memory()
        return {"input_ids": ids, "labels": labels}

    def state_dict(self) -> dict:
        return {"generator": self.gen.get_state(), "batches_yielded": self.batches_yielded}

    def load_state_dict(self, state: dict) -> None:
        self.gen.set_state(state["generator"])
        self.batches_yielded = state.get("batches_yielded", 0)


def phase_weights(phase, names: list[str], sources) -> list[float]:
    """Mixture weights of a training phase in dataset order: the phase's value for a dataset it names, the
    configured weight otherwise (scripts/train.py:613-632, 904-915 of the reference)."""
    configured = [src.weight for src in sources]
    if len(configured) != len(names):
        configured = [1.0] * len(names)
    return [float(phase.dataset_weights.get(name, w)) for name, w in zip(names, configured)]


class Trainer:
    def __init__(self, config: JobConfig, hooks: list | None = None, model=None, dataloader=None,
                 init_dist: bool = True, transport: str | None = None) -> None:
        self.config = config
        tc = config.train
        self.rank, self.local_rank, self.world_size = get_world_info()
        self.mesh = init_distributed(config.distributed, tc.seed) if init_dist else None
        if not init_dist:
            from kempnerforge_b200.parallel.setup import set_seed

            set_seed(tc.seed)
        config.validate(self.world_size)
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.dp_rank, self.dp_size = get_dp_info(self.mesh)
        if self.mesh is None and self.world_size == 1:
            self.dp_rank, self.dp_size = 0, 1
        self.pp_group, self.pp_size, self.pp_rank = mesh_dim(self.mesh, "pp")

        from kempnerforge_b200.resilience import NaNDetector, ShutdownHandler

        self.shutdown = ShutdownHandler(timeout_sec=tc.shutdown_timeout_sec)
        self.nan_detector = NaNDetector(action="warn", max_consecutive=10)

        self.pipeline = None
        self._transport = transport
        self._freeze_stage_idx = -1
        if model is not None:
            self.model = model
        elif config.is_vlm:
            from kempnerforge_b200.parallel.parallel import build_parallel_vlm

            self.model = build_parallel_vlm(config, self.device, self.mesh, step=0, transport=transport)
        elif self.pp_size > 1:
            from kempnerforge_b200.parallel.pipeline_parallel import build_pipeline

            self.pipeline = build_pipeline(config, self.device, self.mesh, transport=transport)
            self.model = self.pipeline.module
        else:
            self.model = build_parallel_model(
                config.model, self.device, self.mesh,
                ac_mode=str(tc.activation_checkpointing), param_dtype=tc.param_dtype,
                fp8=tc.is_fp8, compile_model=False, transport=transport,
                ep_in_dp=config.distributed.ep_in_dp and config.distributed.ep > 1,
                param_sharding=getattr(config.distributed, "param_sharding", None),
            )
        self.engine = getattr(self.model, "_kf_engine", None)
        self.optimizer = build_optimizer(self.model, config.optimizer)
        if isinstance(self.optimizer, FusedAdamW) and self.engine is not None:
            self.optimizer.grad_scale = self.engine.grad_scale
        self.scheduler = build_scheduler(self.optimizer, config.scheduler, tc.max_steps)
        self.step = 0
        self.tokens_seen = 0
        self.phase_idx = -1
        self.phases = config.data.effective_phases()
        self.hook_runner = HookRunner((hooks or []) + load_hooks(tc.hooks))
        self.tracker = MetricsTracker(config.metrics, config.model, num_gpus=self.world_size,
                                      seq_len=tc.seq_len, rank=self.rank)
        self.dataloader = dataloader
        self._data_iter = None
        self.ckpt = None
        self.eval_dataloader = None
        self._loss_acc = torch.zeros(3, dtype=torch.float32, device=self.device)  # loss, grad_norm, finite
        self.completed = False

    # ------------------------------------------------------------------ data
    def _default_dataloader(self):
        from kempnerforge_b200.data import build_train_dataloader, build_vlm_dataloader

        if self.config.is_vlm:
            return build_vlm_dataloader(self.config, self.dp_rank, self.dp_size)
        return build_train_dataloader(self.config, self.dp_rank, self.dp_size)

    # ------------------------------------------------------------------ freeze schedule (vision-language runs)
    def _maybe_advance_freeze_stage(self) -> None:
        """At a stage boundary the set of trainable parameters changes: drain pending communication and
        saves, flip ``requires_grad``, then rebuild the flat groups and the optimizer; moments of parameters
        that stay trainable are carried over by name."""
        vlm = self.config.vlm
        if vlm is None or not vlm.freeze_schedule:
            return
        idx = -1
        for i, stage in enumerate(vlm.freeze_schedule):
            if self.step >= stage.start_step:
                idx = i
        if idx == self._freeze_stage_idx:
            return
        first = self._freeze_stage_idx == -1 and self.step == 0 and idx == -1
        self._freeze_stage_idx = idx
        if first:
            return
        from kempnerforge_b200.checkpoint.manager import load_optimizer_state_dict, optimizer_state_dict
        from kempnerforge_b200.models.vlm import is_encoder_frozen
        from kempnerforge_b200.parallel.parallel import apply_fsdp2
        from kempnerforge_b200.training.freeze import apply_freeze_specs, effective_freeze

        if self.engine is not None:
            self.engine.wait_all()
        if self.ckpt is not None:
            self.ckpt.wait()
        old_state = optimizer_state_dict(self.model, self.optimizer)
        lr_now = [g["lr"] for g in self.optimizer.param_groups]
        specs = effective_freeze(vlm, self.step)
        counts = apply_freeze_specs(self.model, specs, vlm.module_patterns)
        self.model.vision_encoder.train(not is_encoder_frozen(specs))
        log.info("freeze stage %d at step %d: %s", idx, self.step, counts)
        if self.engine is not None:
            self.engine.release()
        apply_fsdp2(self.model, self.mesh, transport=self._transport)
        self.engine = getattr(self.model, "_kf_engine", None)
        self.optimizer = build_optimizer(self.model, self.config.optimizer)
        if isinstance(self.optimizer, FusedAdamW) and self.engine is not None:
            self.optimizer.grad_scale = self.engine.grad_scale
        load_optimizer_state_dict(self.model, self.optimizer, old_state)
        sched_state = self.scheduler.state_dict()
        self.scheduler = build_scheduler(self.optimizer, self.config.scheduler, self.config.train.max_steps)
        self.scheduler.load_state_dict(sched_state)
        for g, lr in zip(self.optimizer.param_groups, lr_now):
            g["lr"] = lr
        if self.ckpt is not None:
            self.ckpt.optimizer = self.optimizer

    def next_batch(self) -> dict[str, torch.Tensor]:
        if self.dataloader is None:
            self.dataloader = self._default_dataloader()
        if self._data_iter is None:
            self._data_iter = iter(self.dataloader)
        try:
            return next(self._data_iter)
        except StopIteration:  # epoch rolled over
            self._data_iter = iter(self.dataloader)
            return next(self._data_iter)

    # ------------------------------------------------------------------ one optimizer step
    def micro_loss(self, batch: dict[str, torch.Tensor]) -> torch.Tensor:
        mc, tc = self.config.model, self.config.train
        model = self.model
        ids = batch["input_ids"]
        labels = batch["labels"]
        doc_ids = batch.get("doc_ids")
        if "pixel_values" in batch:
            pixels = batch["pixel_values"]
            enc_param = next(model.vision_encoder.parameters(), None)
            if enc_param is not None and pixels.dtype != enc_param.dtype:
                pixels = pixels.to(enc_param.dtype)
            return model.compute_loss(pixels, ids, labels, frame_mask=batch.get("frame_mask"),
                                      z_loss_weight=tc.z_loss_weight)
        if hasattr(model, "compute_loss"):
            loss = model.compute_loss(ids, labels, doc_ids=doc_ids, z_loss_weight=tc.z_loss_weight,
                                      chunk_tokens=tc.ce_chunk_size or 4096)
        else:
            from kempnerforge_b200.training.loss import build_loss_fn

            loss = build_loss_fn(tc)(model(ids, doc_ids=doc_ids), labels)
        if mc.is_moe:
            inner = model
            if mc.moe_aux_loss_weight > 0:
                loss = loss + mc.moe_aux_loss_weight * inner.get_moe_aux_loss()
            if mc.moe_router_z_loss_weight > 0:
                loss = loss + mc.moe_router_z_loss_weight * inner.get_moe_router_z_loss()
        return loss

    def train_step(self, batches: list[dict[str, torch.Tensor]] | None = None) -> dict[str, float]:
        """One optimizer step over ``grad_accum_steps`` micro-batches; returns loss / grad_norm / lr / skipped."""
        tc = self.config.train
        accum = tc.grad_accum_steps
        if self.pipeline is not None:
            return self._pipeline_step(batches)
        self.model.train()
        self._loss_acc.zero_()
        if self.config.model.is_moe and hasattr(self.model, "set_moe_step"):
            self.model.set_moe_step(self.step, tc.max_steps)
        per_dataset = self._dataset_metrics_wanted()
        self._dataset_stats = {} if per_dataset else None
        self._text_tokens = None
        for micro in range(accum):
            batch = batches[micro] if batches is not None else self.next_batch()
            batch = _to_device(batch, self.device)
            with maybe_no_sync(self.model, micro, accum):
                if per_dataset and "dataset_idx" in batch:
                    loss = self._micro_loss_with_dataset_stats(batch)
                else:
                    loss = self.micro_loss(batch)
                (loss / accum).backward()
            if "pixel_values" in batch and self._logs_next_step():
                n = (self._vlm_target_labels(batch["labels"]) != -100).sum()
                self._text_tokens = n if self._text_tokens is None else self._text_tokens + n
            self._loss_acc[0] += loss.detach().float() / accum
        if self.engine is not None:
            self.engine.finish_backward()
        grad_norm = clip_grad_norm_(self.model, tc.grad_clip_norm)
        self._loss_acc[1] = grad_norm.to(self._loss_acc.device)
        return self._finish_step()

    def _finish_step(self) -> dict[str, float]:
        acc = self._loss_acc
        acc[2] = torch.isfinite(acc[0]) & torch.isfinite(acc[1])
        if self.world_size > 1 and dist.is_initialized():
            flag = acc[2:3].clone()
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            acc[2] = flag[0]
        loss, grad_norm, finite = (float(x) for x in acc.tolist())  # the step's single host read
        skipped = not self.nan_detector.check_values(loss, grad_norm, bool(finite), self.step)
        lr = self.optimizer.param_groups[0]["lr"]
        if not skipped:
            if self.engine is not None and not isinstance(self.optimizer, FusedAdamW):
                self.engine.apply_grad_scale()
            self.optimizer.step()
            if self.engine is not None:
                self.engine.after_optimizer_step()
            # a skipped (non-finite) step advances neither the optimizer nor the schedule, like the reference's loop
            self.scheduler.step()
            self._apply_phase_lr()
        if self.engine is not None and getattr(self.optimizer, "_kf_engine_bound", None) is not self.engine:
            self.engine.zero_grad()
        self.optimizer.zero_grad(set_to_none=True)   # a bound optimizer resets the engine's flat gradients as well
        return {"loss": loss, "grad_norm": grad_norm, "lr": lr, "skipped": float(skipped)}

    def _pipeline_step(self, batches) -> dict[str, float]:
        tc = self.config.train
        micro = [(_to_device(b, self.device)) for b in (batches or [self.next_batch() for _ in range(tc.grad_accum_steps)])]
        loss = self.pipeline.run_step(micro, z_loss_weight=tc.z_loss_weight)
        if self.engine is not None:
            self.engine.finish_backward()
        grad_norm = self.pipeline.clip_grad_norm(self.model, tc.grad_clip_norm)
        self._loss_acc[0] = loss
        self._loss_acc[1] = grad_norm
        self.pipeline.share_scalars(self._loss_acc)
        return self._finish_step()

    def _native_status(self) -> int:
        """Status word of the native kernel library on this rank's GPU (0 on CPU and when every wait completed)."""
        if self.device.type != "cuda":
            return 0
        from kempnerforge_b200.resilience import check_native_kernel_status

        return check_native_kernel_status()

    def _apply_phase_lr(self) -> None:
        if self.phase_idx >= 0 and self.phases:
            scale = self.phases[self.phase_idx].lr_scale
            if scale != 1.0:
                for g in self.optimizer.param_groups:
                    g["lr"] *= scale

    def _maybe_advance_phase(self) -> None:
        new_idx = -1
        for i, ph in enumerate(self.phases):
            if self.step >= ph.start_step:
                new_idx = i
        if new_idx != self.phase_idx:
            self.phase_idx = new_idx
            if new_idx >= 0:
                ph = self.phases[new_idx]
                log.info("Entering data phase %d at step %d (lr_scale=%s)", new_idx, self.step, ph.lr_scale)
                sampler = getattr(self.dataloader, "sampler", None)
                names = getattr(getattr(self.dataloader, "dataset", None), "dataset_names", None)
                if ph.dataset_weights and names and hasattr(sampler, "update_weights"):
                    sampler.update_weights(phase_weights(ph, names, self.config.data.datasets),
                                           self.config.data.mix_temperature)
                    self._data_iter = None

    # ------------------------------------------------------------------ full run
    def setup_checkpointing(self) -> None:
        from kempnerforge_b200.checkpoint import CheckpointManager
        from kempnerforge_b200.resilience import resolve_resume_path

        cfg = self.config.checkpoint
        stage_group = None
        if self.pp_size > 1 and self.mesh is not None:
            # each pipeline stage writes and reads its own sub-directory, coordinated among the ranks of that stage
            from kempnerforge_b200.parallel.pipeline_parallel import stage_process_group

            stage_group = stage_process_group(self.mesh)
        self.ckpt = CheckpointManager(cfg, self.model, self.optimizer, pp_rank=self.pp_rank if self.pp_size > 1 else None,
                                      process_group=stage_group)
        resume = cfg.load_path or resolve_resume_path(cfg.dir)
        if resume:
            exclude = list(cfg.exclude_from_loading) or None
            freeze_expected = None
            vlm = self.config.vlm
            if vlm is not None:
                # The trainable set at the saved step may differ from the one the model was built with (step 0):
                # move to the saved step's freeze stage first, so the flat groups and the optimizer template hold
                # exactly the parameters whose moments the checkpoint carries; then compare the freeze metadata.
                from kempnerforge_b200.training.freeze import canonical_freeze_meta, effective_freeze

                probe = self.ckpt.peek_saved_step(resume) or 0
                freeze_expected = canonical_freeze_meta(effective_freeze(vlm, probe))
                if vlm.freeze_schedule and probe > 0:
                    self.step = probe
                    self._maybe_advance_freeze_stage()
            self.step, self.tokens_seen, extra = self.ckpt.load(
                path=resume, scheduler=self.scheduler, dataloader=self.dataloader, exclude_keys=exclude,
                vlm_freeze_expected=freeze_expected, allow_fallback=not cfg.load_path)
            self.config.metrics.wandb_run_id = extra.get("wandb_run_id", self.config.metrics.wandb_run_id)
            log.info("Resumed from %s at step=%d", resume, self.step)

    def save_checkpoint(self) -> None:
        if self.ckpt is None:
            return
        extra = {"phase_idx": self.phase_idx, "wandb_run_id": self.tracker.wandb_run_id}
        if self.config.vlm is not None:
            from kempnerforge_b200.training.freeze import canonical_freeze_meta, effective_freeze

            extra["vlm_freeze"] = canonical_freeze_meta(effective_freeze(self.config.vlm, self.step))
        path = self.ckpt.save(self.step, self.tokens_seen, scheduler=self.scheduler, dataloader=self.dataloader,
                              extra=extra)
        self.hook_runner.on_checkpoint_save(self.step, str(path))

    def fit(self) -> dict[str, float]:
        cfg, tc = self.config, self.config.train
        self.shutdown.register()
        if self.dataloader is None:
            self.dataloader = self._default_dataloader()
        self.setup_checkpointing()
        if self.ckpt is not None:
            self.ckpt.apply_dataloader_state(self.dataloader)
        self.tracker.config.wandb_run_id = cfg.metrics.wandb_run_id
        self.tracker.init_backends()
        self._setup_eval()
        from kempnerforge_b200.profiling import build_profiler, print_profiler_summary

        prof = build_profiler(cfg.profiling, self.rank)
        self._maybe_advance_phase()
        self.model.train()
        self.hook_runner.on_train_begin(cfg)
        log.info("Starting training: step=%d, max_steps=%d, world_size=%d, dp_size=%d",
                 self.step, tc.max_steps, self.world_size, self.dp_size)
        if self.step == 0 and cfg.checkpoint.dyn_ckpt_window is not None and cfg.checkpoint.should_save(0):
            self.save_checkpoint()
        if prof is not None:
            prof.start()
        tokens_per_step = tc.batch_size * tc.seq_len * tc.grad_accum_steps * self.dp_size
        last = {"loss": float("nan"), "grad_norm": 0.0, "lr": 0.0}
        stop_reason = None
        while self.step < tc.max_steps:
            self._maybe_advance_freeze_stage()
            self.tracker.start_step()
            out = self.train_step()
            self.step += 1
            if out["skipped"]:
                if self.nan_detector.should_stop:
                    stop_reason = "nan"
                    log.error("Too many consecutive non-finite steps; stopping at step %d", self.step)
                    break
                continue
            last = out
            self.tokens_seen += tokens_per_step
            self._maybe_advance_phase()
            extra = self._moe_metrics() if (self.step % cfg.metrics.log_interval == 0 or self.step == 1) else None
            self.tracker.end_step(self.step, out["loss"], out["grad_norm"], out["lr"], tokens_per_step, extra)
            ctx = StepContext(self.step, out["loss"], out["grad_norm"], out["lr"], self.tokens_seen, self.model,
                              self.optimizer)
            self.hook_runner.on_step_end(ctx)
            if ctx.metrics:
                self.tracker.log_extra(ctx.metrics, self.step)
            ds_metrics = {**self._text_token_metrics(), **self._dataset_metrics()}
            if ds_metrics:
                self.tracker.log_eval(ds_metrics, self.step)
            if any(getattr(h, "should_stop", False) for h in self.hook_runner.hooks):
                stop_reason = "hook"
                log.info("a training hook asked to stop at step %d", self.step)
                break
            if self.step % cfg.metrics.log_interval == 0 or self.step == 1:
                # the step's host read already synchronised: the status word of the native kernels costs one small
                # copy here.  Non-zero = a bounded device-side wait gave up (the kernel returned without its result).
                word = self._native_status()
                if word:
                    stop_reason = "kernel_status"
                    log.error("native kernel status word is %d at step %d (a device-side wait ran out); stopping", word, self.step)
                    break
            if tc.nccl_health_check_interval > 0 and self.step % tc.nccl_health_check_interval == 0:
                from kempnerforge_b200.resilience import check_nccl_health

                if not check_nccl_health(timeout_sec=10.0):
                    stop_reason = "comm"
                    log.error("communication health check failed at step %d", self.step)
                    break
            if self.eval_dataloader is not None and self.step % cfg.eval.interval == 0:
                self._run_eval()
            if prof is not None:
                prof.step()
            if self.ckpt is not None and cfg.checkpoint.should_save(self.step):
                self.save_checkpoint()
            if self.shutdown.should_shutdown():
                log.warning("Shutdown requested at step %d — saving emergency checkpoint", self.step)
                self.save_checkpoint()
                stop_reason = "signal"
                break
        else:
            self.completed = True
        if prof is not None:
            prof.stop()
            if self.rank == 0:
                print_profiler_summary(prof, cfg.profiling.trace_dir)
        if self.completed and self.ckpt is not None and not cfg.checkpoint.should_save(self.step):
            self.save_checkpoint()
        if self.ckpt is not None:
            self.ckpt.wait()
        log.info("Training complete: %d steps, %s tokens", self.step, f"{self.tokens_seen:,}")
        self.hook_runner.on_train_end(self.step, self.tokens_seen)
        self.tracker.close()
        self.shutdown.unregister()
        return {**last, "step": self.step, "tokens_seen": self.tokens_seen, "stop_reason": stop_reason}

    # ------------------------------------------------------------------ per-dataset metrics of mixture runs
    def _mixture_names(self) -> list[str] | None:
        return getattr(getattr(self.dataloader, "dataset", None), "dataset_names", None)

    def _logs_next_step(self) -> bool:
        nxt = self.step + 1
        return nxt % self.config.metrics.log_interval == 0 or nxt == 1

    def _vlm_target_labels(self, labels: torch.Tensor) -> torch.Tensor:
        """The label positions the vision-language wrapper scores (all but the first when it shifts them)."""
        return labels[:, 1:] if getattr(self.model, "shift_labels", True) else labels

    def _text_token_metrics(self) -> dict[str, float]:
        """``data/text_tokens_trained``: text positions that carried a loss in the logged step, summed over ranks
        (image prefix, padding and masked prompt tokens excluded); vision-language runs only."""
        n = getattr(self, "_text_tokens", None)
        if n is None:
            return {}
        n = n.to(torch.int64).reshape(1)
        if self.world_size > 1 and dist.is_initialized():
            dist.all_reduce(n)
        return {"data/text_tokens_trained": float(n.item())}

    def _dataset_metrics_wanted(self) -> bool:
        """True on the steps whose metrics are logged, for a dataset mixture, outside pipeline / vocabulary-parallel
        runs (there the final hidden states and the head are not on one rank)."""
        if not self._logs_next_step():
            return False
        model = self.model
        return (self._mixture_names() is not None and self.pipeline is None and getattr(model, "norm", None) is not None
                and getattr(getattr(model, "output_head", None), "tp", None) is None)

    def _micro_loss_with_dataset_stats(self, batch) -> torch.Tensor:
        """The ordinary micro-batch loss; also records, per source dataset of the mixture, the mean loss of its rows
        and their token count (kempnerforge scripts/train.py:822-839 computes the same from the logits).  The final
        hidden states are captured by a forward hook and pushed through the head once more without gradients, in
        chunks, so the training path itself is unchanged."""
        from kempnerforge_b200.ops import functional as F

        captured = []
        handle = self.model.norm.register_forward_hook(lambda _m, _i, out: captured.append(out.detach()))
        try:
            loss = self.micro_loss(batch)
        finally:
            handle.remove()
        if captured:
            hidden, labels, ds_idx = captured[0], batch["labels"], batch["dataset_idx"]
            weight = self.model.output_head.proj.weight
            seq = labels.shape[1]
            with torch.no_grad():
                for i, name in enumerate(self._mixture_names()):
                    rows = ds_idx == i
                    n_rows = int(rows.sum())
                    if n_rows == 0:
                        continue
                    ds_loss = F.linear_cross_entropy(hidden[rows], weight, labels[rows])
                    acc = self._dataset_stats.setdefault(name, [0.0, 0, 0])
                    acc[0] += float(ds_loss)
                    acc[1] += 1
                    acc[2] += n_rows * seq
        return loss

    def _dataset_metrics(self) -> dict[str, float]:
        stats = getattr(self, "_dataset_stats", None) or {}
        out = {f"loss/{name}": total / max(1, count) for name, (total, count, _) in stats.items()}
        out.update({f"data/{name}/tokens": float(tokens) for name, (_, _, tokens) in stats.items()})
        return out

    # ------------------------------------------------------------------ helpers
    def _moe_metrics(self) -> dict[str, float] | None:
        if not self.config.model.is_moe or not hasattr(self.model, "get_expert_counts"):
            return None
        counts = self.model.get_expert_counts()
        if not counts:
            return None
        stacked = torch.stack([c.float() for c in counts.values()])
        balance = (stacked.min(dim=1).values / stacked.max(dim=1).values.clamp_min(1)).mean()
        vals = torch.stack([self.model.get_moe_aux_loss().float().reshape(()),
                            self.model.get_moe_router_z_loss().float().reshape(()), balance]).tolist()
        return {"moe/aux_loss": vals[0], "moe/router_z_loss": vals[1], "moe/expert_balance": vals[2]}

    def _setup_eval(self) -> None:
        from kempnerforge_b200.training.eval import build_eval_dataloader, should_build_eval_dataloader

        if should_build_eval_dataloader(self.config):
            self.eval_dataloader = build_eval_dataloader(self.config, self.dp_rank, self.dp_size)

    def _run_eval(self) -> None:
        from kempnerforge_b200.training.eval import run_eval

        sf = self.optimizer if hasattr(self.optimizer, "eval_params") else None
        if sf is not None:
            sf.eval_params()
        metrics = run_eval(self.model, self.eval_dataloader, self.config, self.device)
        if sf is not None:
            sf.train_params()
        self.tracker.log_eval(metrics, self.step)
        self.hook_runner.on_eval_end(metrics, self.step)
        self.model.train()
