"""Evaluation loop: mean loss and perplexity over a fixed number of held-out batches.

Parity: kempnerforge/training/eval.py:25-149 (``should_build_eval_dataloader`` — evaluation is off for
vision-language runs and without a source; metrics ``eval/loss`` and ``eval/perplexity = exp(min(loss, 20))``;
all data-parallel ranks average their losses).
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist


def should_build_eval_dataloader(config, is_vlm: bool | None = None):
    """``should_build_eval_dataloader(job_config)`` -> bool.  The flag form ``(eval_enabled, is_vlm)`` returns
    ``(build, warn_that_vlm_eval_is_skipped)`` (kempnerforge/training/eval.py:25-40)."""
    if isinstance(config, bool):
        return (False, True) if config and is_vlm else (config, False)
    ec = config.eval
    if not ec.enabled or getattr(config, "is_vlm", False):
        return False
    return bool(ec.dataset_path or ec.hf_dataset_name)


def build_eval_dataloader(config, dp_rank: int = 0, dp_size: int = 1):
    from kempnerforge_b200.data import DistributedSampler, HuggingFaceDataset, MemoryMappedDataset, StatefulDataLoader

    ec, tc, dc = config.eval, config.train, config.data
    window = tc.seq_len + 1
    if ec.dataset_path:
        ds = MemoryMappedDataset(ec.dataset_path, window, ec.file_pattern)
    else:
        ds = HuggingFaceDataset(ec.hf_dataset_name, tc.seq_len, dc.tokenizer_path, ec.hf_dataset_config,
                                ec.hf_dataset_split, dc.hf_dataset_text_field)
    sampler = DistributedSampler(len(ds), dp_size, dp_rank, shuffle=False, seed=0, drop_last=True)
    return StatefulDataLoader(ds, tc.batch_size, sampler, 0, False, None, True)


@torch.no_grad()
def run_eval(model, dataloader, config, device, pipeline=None, *, eval_steps: int | None = None, pp_schedule=None,
             **_) -> dict[str, float]:
    """Mean loss and perplexity over ``config.eval.steps`` batches (the loader restarts when it runs out).

    ``config`` may instead be a loss function ``(logits, labels) -> scalar``, with the number of batches as the next
    positional argument or ``eval_steps=`` and a pipeline runner as ``pp_schedule=``
    (kempnerforge/training/eval.py:43-130).
    """
    loss_fn = None
    if callable(config) and not hasattr(config, "eval"):
        loss_fn = config
        if isinstance(pipeline, int):
            eval_steps, pipeline = pipeline, None
        pipeline = pipeline if pipeline is not None else pp_schedule
        if eval_steps is None:
            raise TypeError("run_eval with a loss function needs eval_steps")
    steps = eval_steps if eval_steps is not None else config.eval.steps
    was_training = model.training
    model.eval()
    total = torch.zeros(2, dtype=torch.float64, device=device)
    it = iter(dataloader)
    for _ in range(steps):
        try:
            batch = next(it)
        except StopIteration:
            it = iter(dataloader)
            try:
                batch = next(it)
            except StopIteration:
                break
        ids, labels = batch["input_ids"].to(device), batch["labels"].to(device)
        if pipeline is not None:
            loss = pipeline.eval_loss(ids, labels)
        elif loss_fn is not None:
            loss = loss_fn(model(ids), labels)
        elif hasattr(model, "compute_loss"):
            loss = model.compute_loss(ids, labels, doc_ids=batch.get("doc_ids"))
        else:
            from kempnerforge_b200.training.loss import cross_entropy

            loss = cross_entropy(model(ids), labels)
        total[0] += loss.double()
        total[1] += 1
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        buf = total.float() if device.type == "cpu" else total
        dist.all_reduce(buf)
        total = buf.double()
    mean = (total[0] / total[1].clamp_min(1)).item()
    if was_training:
        model.train()
    return {"eval/loss": mean, "eval/perplexity": math.exp(min(mean, 20.0))}
