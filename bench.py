#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B-shape pre-training throughput (tokens/s, whole job) on N B200s.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...        (the unmodified reference package from baseline/_ref)

Config: dim 4096, 32 layers, 32 query / 8 KV heads, SwiGLU 14336, vocab 128256, RoPE theta 5e5, bf16,
full activation checkpointing, fused AdamW (lr 3e-4, wd 0.1), cosine LR, sequence 4096, micro-batch 2 per
GPU, sharded data parallel over all GPUs, synthetic uniform tokens, random N(0, 0.02) weights.

Two timed regions, both through ``Trainer.train_step`` (forward, backward, gradient reduction, clipping,
optimizer step, LR schedule; one host read of loss/grad-norm per step):
  value : batches already resident on the device; CUDA events, max over ranks
  e2e   : every step copies its batch from pinned host memory and reads the loss back
Weak scaling: per-GPU work is fixed.  The working set (16 GB of weights, 16 GB of gradients, 32 GB of
optimizer state, activations) is far larger than the 126 MB L2, so no explicit flush is needed.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H200_PUBLISHED_TOKS = {1: 10471.0, 2: 18728.0, 4: 38983.0}  # tokens/s the reference publishes for H200 (its FSDP rows), by GPU count
MODELS = {
    "llama3_8b": dict(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, vocab_size=128256,
                      ffn_hidden_dim=14336, max_seq_len=4096, rope_theta=500000.0),
    # 13B shape of the tensor-parallel rows (dim 5120, 40 layers, ffn 13824)
    "llama_13b": dict(dim=5120, n_layers=40, n_heads=40, n_kv_heads=8, vocab_size=128256, ffn_hidden_dim=13824,
                      max_seq_len=4096, rope_theta=500000.0),
    # MoE: softmax top-2 over 8 experts of 5632, every layer
    "moe_8x": dict(dim=2048, n_layers=24, n_heads=16, n_kv_heads=16, vocab_size=102400, ffn_hidden_dim=5632,
                   max_seq_len=4096, rope_theta=500000.0, num_experts=8, moe_top_k=2, moe_router="softmax_topk",
                   moe_packed_experts=True),
    # fine-grained MoE with DeepSeek-V3-style routing: 64 routed experts of 1408 (top-6) + 2 shared, sigmoid router with
    # bias balancing and router z-loss, first layer dense (hidden 10944)
    "moe_fine": dict(dim=2048, n_layers=24, n_heads=16, n_kv_heads=16, vocab_size=102400, ffn_hidden_dim=10944,
                     max_seq_len=4096, rope_theta=500000.0, num_experts=64, moe_top_k=6, moe_router="sigmoid_topk",
                     moe_shared_experts=2, moe_router_z_loss_weight=1e-3, moe_first_k_dense=1,
                     moe_expert_ffn_multiplier=1408.0 / 10944.0, moe_packed_experts=True),
    # small shapes for quick functional checks of this script (not benchmark numbers)
    "tiny_moe": dict(dim=512, n_layers=4, n_heads=8, n_kv_heads=2, vocab_size=4096, ffn_hidden_dim=1536,
                     max_seq_len=512, rope_theta=500000.0, num_experts=8, moe_top_k=2, moe_router="sigmoid_topk",
                     moe_shared_experts=1, moe_router_z_loss_weight=1e-3, moe_first_k_dense=1,
                     moe_expert_ffn_multiplier=0.25, moe_packed_experts=True),
    "tiny": dict(dim=512, n_layers=4, n_heads=8, n_kv_heads=2, vocab_size=4096, ffn_hidden_dim=1536,
                 max_seq_len=512, rope_theta=500000.0),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--model", default="llama3_8b", choices=sorted(MODELS))
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--transport", default=None)
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree (data parallel over the rest)")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel degree")
    ap.add_argument("--ep-in-dp", action="store_true", help="experts sharded over the data-parallel ranks (ours only)")
    ap.add_argument("--pp", type=int, default=1, help="pipeline stages (1F1B over --micro-batches)")
    ap.add_argument("--micro-batches", type=int, default=1, help="micro-batches per optimizer step (gradient accumulation)")
    ap.add_argument("--fp8", action="store_true", help="float8 Linear layers (tensorwise scaling)")
    ap.add_argument("--optimizer", default="adamw", choices=("adamw", "muon"))
    ap.add_argument("--param-sharding", default="resident", choices=("auto", "resident", "sharded"),
                    help="data-parallel memory plan (ours only): whole parameters on every rank, or ZeRO-3")
    return ap.parse_args()


def mesh_dims(args, world: int) -> tuple[dict, int, str]:
    """[distributed] fields, number of distinct batches per step, and a label such as "tp2xdp4"."""
    if args.ep > 1 and args.ep_in_dp:
        return {"ep": args.ep, "ep_in_dp": True, "dp_shard": world}, world, f"ep{args.ep}-in-dp{world}"
    dp = world // (args.tp * args.ep * args.pp)
    dims = {"dp_shard": dp}
    label = f"dp{dp}"
    if args.pp > 1:
        dims["pp"] = args.pp
        dims["pp_schedule"] = "1f1b"
    if args.tp > 1:
        dims["tp"] = args.tp
        label = f"tp{args.tp}x" + label
    if args.ep > 1:
        dims["ep"] = args.ep
        label = f"ep{args.ep}x" + label
    if args.pp > 1:
        label = f"pp{args.pp}x" + label
    return dims, dp, label


class ClockSampler:
    """Samples SM clocks and throttle reasons of the local GPU with nvidia-smi during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    return rank, local, world


def timed_region(torch, dist, world, run_step, steps):
    """barrier + synchronize, K steps between CUDA events, synchronize + barrier; returns max-over-ranks ms/step."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    last = None
    for i in range(steps):
        last = run_step(i)
    end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - t0
    ms = torch.tensor([start.elapsed_time(end) / steps], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item()), wall, last


# --------------------------------------------------------------------------- our framework
def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from kempnerforge_b200.config import config_from_dict
    from kempnerforge_b200.metrics.mfu import compute_mfu
    from kempnerforge_b200.ops import cuda as kcuda
    from kempnerforge_b200.ops.build import build
    from kempnerforge_b200.training.trainer import Trainer

    rank, local, world = dist_env()
    if rank == 0:
        build()
    shape = dict(MODELS[args.model])
    seq = args.seq_len or shape["max_seq_len"]
    cfg = config_from_dict({
        "model": shape,
        "train": {"batch_size": args.batch_size, "seq_len": seq, "max_steps": 1000,
                  "grad_accum_steps": args.micro_batches, "mixed_precision": "fp8" if args.fp8 else "bf16",
                  "activation_checkpointing": "full", "compile_model": False, "grad_clip_norm": 1.0, "seed": 0},
        "optimizer": {"name": args.optimizer, "lr": 3e-4, "weight_decay": 0.1, "fused": True},
        "scheduler": {"name": "cosine", "warmup_steps": 10},
        "distributed": {**mesh_dims(args, world)[0], "param_sharding": args.param_sharding},
        "metrics": {"log_interval": 1000},
        "data": {"pin_memory": True},
    })
    _, n_batches, mesh_label = mesh_dims(args, world)
    trainer = Trainer(cfg, transport=args.transport)
    dev = trainer.device
    vocab = shape["vocab_size"]
    gen = torch.Generator().manual_seed(1234 + trainer.dp_rank)  # ranks of one TP / EP group share their batch

    def host_micro():
        tok = torch.randint(0, vocab, (args.batch_size, seq + 1), generator=gen)
        return {"input_ids": tok[:, :-1].contiguous().pin_memory(), "labels": tok[:, 1:].contiguous().pin_memory()}

    def host_batch():  # one optimizer step: --micro-batches micro-batches
        return [host_micro() for _ in range(args.micro_batches)]

    def on_device(step_batches):
        return [{k: v.to(dev) for k, v in mb.items()} for mb in step_batches]

    # a different random batch for every step, so nothing can be memorised
    warm = [on_device(host_batch()) for _ in range(args.warmup)]
    dev_batches = [on_device(host_batch()) for _ in range(args.steps)]
    for b in warm:
        trainer.train_step(b)
    status = kcuda.read_status()
    if status != 0:
        raise RuntimeError(f"native kernel wait status {status} during warm-up")

    sampler = ClockSampler(local)
    launches0 = kcuda.LAUNCH_COUNT
    ms, wall, last = timed_region(torch, dist, world, lambda i: trainer.train_step(dev_batches[i]), args.steps)
    launches = kcuda.LAUNCH_COUNT - launches0
    clocks = sampler.stop()

    host_batches = [host_batch() for _ in range(args.steps)]
    h2d = sum(v.numel() * v.element_size() for mb in host_batches[0] for v in mb.values())
    ms_e2e, _, last_e2e = timed_region(torch, dist, world,
                                       lambda i: trainer.train_step(host_batches[i]), args.steps)
    n_batches *= args.micro_batches
    tokens_per_step = args.batch_size * seq * n_batches
    value = tokens_per_step / (ms / 1e3)
    e2e = tokens_per_step / (ms_e2e / 1e3)
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peaks = json.load(fh)
    except OSError:
        pass
    mfu_nominal = compute_mfu(cfg.model, value, world, 2250.0, seq)
    mfu_measured = compute_mfu(cfg.model, value, world, peaks.get("bf16_tflops", 1590.0), seq)
    base = H200_PUBLISHED_TOKS.get(world)
    return {
        "metric": f"{args.model}_train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": (value / base) if (base and args.model == "llama3_8b" and mesh_label == f"dp{world}") else None,
        "dtype": "fp8 (E4M3 / E5M2 linear layers, bf16 elsewhere)" if args.fp8 else "bf16",
        "data": "synthetic uniform tokens, random-init weights", "impl": "ours",
        "config": {"model": args.model, "global_batch": args.batch_size * n_batches, "seq_len": seq,
                   "parallelism": mesh_label, "activation_checkpointing": "full",
                   "optimizer": "adamw_fused" if args.optimizer == "adamw" else "muon (Newton-Schulz 5) + adamw"},
        "notes": {"micro_batches": args.micro_batches, "l2": "working set (>60 GB) far exceeds L2; no flush needed",
                  "param_sharding": type(trainer.engine).__name__ if trainer.engine is not None else None,
                  "engine_memory_gb": (trainer.engine.memory_report() if hasattr(trainer.engine, "memory_report") else None)},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 12},
        "gpu_launches": launches,
        "mfu_of_nominal_2250": mfu_nominal, "mfu_of_measured_cublas": mfu_measured,
        "loss": last["loss"] if last else None, "wall_s_timed": wall,
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
        "device_mem_used_gb": device_mem_used_gb(torch),
    }


def device_mem_used_gb(torch) -> float:
    """Memory in use on this GPU as the driver sees it (total - free): includes symmetric-memory buffers, which the
    caching allocator's statistics do not count."""
    free, total = torch.cuda.mem_get_info()
    return (total - free) / 2**30


# --------------------------------------------------------------------------- reference framework
def run_reference(args) -> dict:
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "kempnerforge")):
        return {"impl": "reference", "unavailable": "reference package is not installed under baseline/_ref"}
    sys.path.insert(0, ref_root)
    sys.modules.pop("kempnerforge", None)
    import torch
    import torch.distributed as dist

    try:
        from kempnerforge.config.schema import JobConfig  # noqa: F401
        from kempnerforge.config.loader import load_config
        from kempnerforge.distributed import clip_grad_norm_, init_distributed
        from kempnerforge.distributed.parallel import build_parallel_model
        from kempnerforge.training.loss import build_loss_fn
        from kempnerforge.training.optimizer import build_optimizer
        from kempnerforge.training.scheduler import build_scheduler
    except Exception as exc:  # e.g. a hard dependency that is not in the image
        return {"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"[:300]}

    rank, local, world = dist_env()
    shape = MODELS[args.model]
    if args.ep_in_dp:
        return {"impl": "reference", "unavailable": "the reference cannot shard experts over its data-parallel ranks"}
    if args.fp8:
        return {"impl": "reference", "unavailable": "the reference's float8 path needs torchao, which is not installed"}
    if args.pp > 1 or args.micro_batches > 1 or args.optimizer != "adamw":
        return {"impl": "reference", "unavailable": "this harness drives the reference's plain text step only "
                "(no pipeline schedule / accumulation / Muon)"}
    notes = []
    if shape.get("moe_first_k_dense"):
        # the reference can only place MoE layers by frequency: every layer becomes an MoE layer there
        shape = {k: v for k, v in shape.items() if k != "moe_first_k_dense"}
        notes.append("reference has no moe_first_k_dense: all layers are MoE layers in this arm")
    seq = args.seq_len or shape["max_seq_len"]
    overrides = [f"--model.{k}={v}" for k, v in shape.items()] + [
        f"--train.batch_size={args.batch_size}", f"--train.seq_len={seq}", "--train.max_steps=1000",
        "--train.grad_accum_steps=1", "--train.mixed_precision=bf16", "--train.activation_checkpointing=full",
        "--train.compile_model=true", "--train.grad_clip_norm=1.0", "--train.seed=0",
        "--optimizer.name=adamw", "--optimizer.lr=3e-4", "--optimizer.weight_decay=0.1", "--optimizer.fused=true",
        "--scheduler.name=cosine", "--scheduler.warmup_steps=10",
    ]
    dims, n_batches, mesh_label = mesh_dims(args, world)
    overrides += [f"--distributed.{k}={v}" for k, v in dims.items()]
    if shape.get("num_experts"):
        overrides = [o for o in overrides if o != "--train.compile_model=true"] + ["--train.compile_model=false"]
    config = load_config(None, overrides)
    tc, mc = config.train, config.model
    device_mesh = init_distributed(config.distributed, seed=tc.seed)
    config.validate(world)
    device = torch.device(f"cuda:{local}")
    model = build_parallel_model(mc, device, device_mesh, ac_mode=tc.activation_checkpointing,
                                 param_dtype=tc.param_dtype, compile_model=tc.compile_model, fp8=False)
    optimizer = build_optimizer(model, config.optimizer)
    scheduler = build_scheduler(optimizer, config.scheduler, max_steps=tc.max_steps)
    loss_fn = build_loss_fn(tc)
    model.train()
    from kempnerforge.distributed.utils import get_dp_info

    dp_rank = get_dp_info(device_mesh)[0] if device_mesh is not None else 0
    gen = torch.Generator().manual_seed(1234 + dp_rank)

    def host_batch():
        tok = torch.randint(0, mc.vocab_size, (args.batch_size, seq + 1), generator=gen)
        return tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()

    def step(ids, labels):
        # the reference's text training step (scripts/train.py: forward, loss, backward, loss.item(),
        # clip_grad_norm_, grad_norm.item(), optimizer.step, scheduler.step, zero_grad)
        ids, labels = ids.to(device, non_blocking=True), labels.to(device, non_blocking=True)
        logits = model(ids)
        loss = loss_fn(logits, labels)
        loss.backward()
        loss_val = loss.item()
        grad_norm = clip_grad_norm_(model, tc.grad_clip_norm)
        _ = grad_norm.item() if isinstance(grad_norm, torch.Tensor) else grad_norm
        optimizer.step()
        scheduler.step()
        optimizer.zero_grad()
        return {"loss": loss_val}

    warm = [tuple(t.to(device) for t in host_batch()) for _ in range(args.warmup)]
    dev_batches = [tuple(t.to(device) for t in host_batch()) for _ in range(args.steps)]
    for b in warm:
        step(*b)
    sampler = ClockSampler(local)
    ms, wall, last = timed_region(torch, dist, world, lambda i: step(*dev_batches[i]), args.steps)
    clocks = sampler.stop()
    host_batches = [host_batch() for _ in range(args.steps)]
    h2d = sum(t.numel() * t.element_size() for t in host_batches[0])
    ms_e2e, _, _ = timed_region(torch, dist, world, lambda i: step(*host_batches[i]), args.steps)
    tokens_per_step = args.batch_size * seq * n_batches
    value = tokens_per_step / (ms / 1e3)
    base = H200_PUBLISHED_TOKS.get(world)
    return {
        "metric": f"{args.model}_train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": (value / base) if (base and args.model == "llama3_8b" and mesh_label == f"dp{world}") else None,
        "dtype": "bf16", "data": "synthetic uniform tokens, random-init weights", "impl": "reference",
        "config": {"model": args.model, "global_batch": args.batch_size * n_batches, "seq_len": seq,
                   "parallelism": mesh_label, "activation_checkpointing": "full", "optimizer": "adamw_fused"},
        "notes": {"compile_model": not shape.get("num_experts"), "remarks": notes},
        "clocks": clocks,
        "e2e": {"value": tokens_per_step / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8},
        "gpu_launches": 0, "loss": last["loss"] if last else None, "wall_s_timed": wall,
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30,
        "device_mem_used_gb": device_mem_used_gb(torch),
    }


def main() -> int:
    args = parse_args()
    rank, _, world = dist_env()
    if world != args.gpus and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE={world}; using the launcher's world size", file=sys.stderr)
    try:
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    except Exception as exc:
        if args.impl == "reference":
            result = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}
        else:
            raise
    if rank == 0:
        print(json.dumps(result), flush=True)
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
