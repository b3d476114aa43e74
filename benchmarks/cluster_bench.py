"""Cluster benchmark driver: runs a named matrix of training experiments through ``scripts/train.py``
and tabulates tokens/s, MFU, step time and peak memory from the trainer's own log lines.

    python benchmarks/cluster_bench.py mfu_scaling --steps 30            # every experiment that fits
    python benchmarks/cluster_bench.py moe_ep --only 01 05 --dry-run     # print the commands only
    python benchmarks/cluster_bench.py moe_packed --results-dir out/moe_packed

An experiment needs ``gpus`` GPUs. With 8 or fewer it runs under torchrun on this node; larger ones
need a SLURM allocation (``srun`` with 8 tasks per node) and are skipped when there is none or it is
too small. All experiments start from ``configs/train/debug.toml`` plus CLI overrides, as the
reference's drivers do (benchmarks/mfu_scaling/mfu_bench.sh:16-23,74-129,
benchmarks/moe_expert_parallel/moe_ep_bench.sh, benchmarks/moe_packed/moe_packed_bench.sh); the
matrices below are the same experiments re-packed for 8-GPU NVSwitch nodes.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import shlex
import subprocess
import sys
import time
from dataclasses import dataclass

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GPUS_PER_NODE = 8

M7B = ("--model.dim=4096 --model.n_layers=32 --model.n_heads=32 --model.n_kv_heads=8 --model.vocab_size=128256 "
       "--model.ffn_hidden_dim=14336 --model.max_seq_len=4096")
M13B = ("--model.dim=5120 --model.n_layers=40 --model.n_heads=40 --model.n_kv_heads=8 --model.vocab_size=128256 "
        "--model.ffn_hidden_dim=13824 --model.max_seq_len=4096")
M70B = ("--model.dim=8192 --model.n_layers=80 --model.n_heads=64 --model.n_kv_heads=8 --model.vocab_size=128256 "
        "--model.ffn_hidden_dim=28672 --model.max_seq_len=4096")
MOE = ("--model.dim=2048 --model.n_layers=24 --model.n_heads=16 --model.n_kv_heads=4 --model.vocab_size=128256 "
       "--model.max_seq_len=4096 --model.num_experts=8 --model.moe_top_k=2 --model.moe_frequency=1 "
       "--model.ffn_hidden_dim=5632")
TRAIN = ("--train.seq_len=4096 --train.mixed_precision=bf16 --train.activation_checkpointing=full "
         "--optimizer.fused=true --metrics.log_interval=5 --checkpoint.interval=1000000")


@dataclass
class Experiment:
    tag: str
    gpus: int
    args: str


def _dense(tag, gpus, model, bs, accum, **dist) -> Experiment:
    d = " ".join(f"--distributed.{k}={v}" for k, v in dist.items())
    return Experiment(tag, gpus, f"{model} {TRAIN} --train.batch_size={bs} --train.grad_accum_steps={accum} {d}")


def _moe(tag, gpus, bs, accum, ac, extra="", **dist) -> Experiment:
    d = " ".join(f"--distributed.{k}={v}" for k, v in dist.items())
    t = TRAIN.replace("activation_checkpointing=full", f"activation_checkpointing={ac}")
    return Experiment(tag, gpus, f"{MOE} {t} --train.batch_size={bs} --train.grad_accum_steps={accum} {extra} {d}")


MATRICES: dict[str, list[Experiment]] = {
    "mfu_scaling": [
        _dense("01_1gpu_7b", 1, M7B, 2, 4, dp_shard=1),
        _dense("02_2gpu_7b_fsdp2", 2, M7B, 2, 4, dp_shard=2),
        _dense("03_2gpu_7b_tp2", 2, M7B, 4, 2, tp=2, dp_shard=1),
        _dense("04_4gpu_7b_fsdp4", 4, M7B, 4, 2, dp_shard=4),
        _dense("05_4gpu_7b_tp4", 4, M7B, 4, 2, tp=4, dp_shard=1),
        _dense("06_4gpu_7b_tp2_fsdp2", 4, M7B, 4, 2, tp=2, dp_shard=2),
        _dense("07_8gpu_7b_fsdp8", 8, M7B, 2, 1, dp_shard=8),
        _dense("08_8gpu_7b_tp4_fsdp2", 8, M7B, 4, 2, tp=4, dp_shard=2),
        _dense("09_8gpu_13b_fsdp8", 8, M13B, 4, 4, dp_shard=8),
        _dense("10_8gpu_13b_tp4_fsdp2", 8, M13B, 4, 4, tp=4, dp_shard=2),
        _dense("11_16gpu_7b_tp4_fsdp4", 16, M7B, 4, 2, tp=4, dp_shard=4),
        _dense("12_16gpu_13b_tp4_fsdp4", 16, M13B, 4, 4, tp=4, dp_shard=4),
        _dense("13_32gpu_7b_tp4_fsdp8", 32, M7B, 4, 2, tp=4, dp_shard=8),
        _dense("14_32gpu_13b_tp4_fsdp8", 32, M13B, 4, 4, tp=4, dp_shard=8),
        _dense("15_32gpu_70b_tp4_fsdp8", 32, M70B, 2, 4, tp=4, dp_shard=8),
    ],
    "moe_ep": [
        _moe("01_ep2_tp4_fsdp4_bs8_fullac", 32, 8, 1, "full", tp=4, ep=2, dp_shard=4),
        _moe("02_ep2_tp4_fsdp4_bs2_fullac", 32, 2, 4, "full", tp=4, ep=2, dp_shard=4),
        _moe("03_ep2_tp4_fsdp4_bs12_fullac", 32, 12, 1, "full", tp=4, ep=2, dp_shard=4),
        _moe("04_ep2_tp4_fsdp4_bs1_selectiveac", 32, 1, 8, "selective", tp=4, ep=2, dp_shard=4),
        _moe("05_noep_tp4_fsdp8_bs8_fullac", 32, 8, 1, "full", tp=4, ep=1, dp_shard=8),
        _moe("06_noep_tp4_fsdp8_bs8_selectiveac", 32, 8, 1, "selective", tp=4, ep=1, dp_shard=8),
        _moe("07_1node_ep8_in_dp_bs4_fullac", 8, 4, 1, "full", extra="--distributed.ep_in_dp=true", ep=8, dp_shard=8),
        _moe("08_1node_ep2_fsdp4_bs4_fullac", 8, 4, 1, "full", ep=2, dp_shard=4),
    ],
    "moe_packed": [
        _moe(f"{i:02d}_E{e}_{'packed' if packed else 'unpacked'}", 4, 4, 1, "full",
             extra=f"--model.num_experts={e} --model.moe_packed_experts={'true' if packed else 'false'}", dp_shard=4)
        for i, (e, packed) in enumerate([(8, False), (8, True), (16, False), (16, True), (32, False), (32, True),
                                         (64, False), (64, True)], start=1)
    ],
}

_STEP = re.compile(r"\[step (\d+)\].*?tok/s=([\d,]+).*?mfu=([\d.]+)%.*?mem=([\d.]+)/.*?step_time=([\d.]+)s")


def parse_log(text: str, skip: int = 2) -> dict | None:
    """Mean of the logged steps after the first ``skip`` (warm-up) log lines."""
    rows = [(int(m[1]), float(m[2].replace(",", "")), float(m[3]), float(m[4]), float(m[5]))
            for m in _STEP.finditer(text)]
    rows = rows[skip:] or rows[-1:]
    if not rows:
        return None
    n = len(rows)
    return {"last_step": rows[-1][0], "tokens_per_sec": sum(r[1] for r in rows) / n, "mfu_pct": sum(r[2] for r in rows) / n,
            "peak_mem_gb": max(r[3] for r in rows), "step_time_s": sum(r[4] for r in rows) / n}


def launch_command(exp: Experiment, steps: int, port: int, extra: str) -> list[str] | None:
    tail = ["scripts/train.py", "configs/train/debug.toml", *shlex.split(exp.args), f"--train.max_steps={steps}",
            *shlex.split(extra)]
    if exp.gpus <= GPUS_PER_NODE:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={exp.gpus}",
                "--master-addr", "127.0.0.1", "--master-port", str(port), *tail]
    nodes = exp.gpus // GPUS_PER_NODE
    if int(os.environ.get("SLURM_NNODES", "0")) < nodes:
        return None
    return ["srun", f"--nodes={nodes}", f"--ntasks={exp.gpus}", f"--gpus-per-node={GPUS_PER_NODE}", "--kill-on-bad-exit=1",
            os.path.join(ROOT, "scripts/slurm/_run_training.sh"), *tail[1:]]


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="run a benchmark matrix through scripts/train.py")
    ap.add_argument("matrix", choices=sorted(MATRICES))
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--only", nargs="*", default=None, help="tag prefixes to run")
    ap.add_argument("--results-dir", default=None)
    ap.add_argument("--extra", default="", help="overrides appended to every experiment (e.g. data arguments)")
    ap.add_argument("--max-gpus", type=int, default=None, help="skip experiments that need more")
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    out_dir = args.results_dir or os.path.join(ROOT, "benchmarks", "results", args.matrix)
    os.makedirs(out_dir, exist_ok=True)
    summary = []
    for i, exp in enumerate(MATRICES[args.matrix]):
        if args.only and not any(exp.tag.startswith(p) for p in args.only):
            continue
        if args.max_gpus is not None and exp.gpus > args.max_gpus:
            continue
        cmd = launch_command(exp, args.steps, 29700 + i, args.extra)
        if cmd is None:
            print(f"-- {exp.tag}: needs {exp.gpus} GPUs, no SLURM allocation of that size; skipped")
            continue
        print(f">> {exp.tag} ({exp.gpus} GPUs)\n   {' '.join(shlex.quote(c) for c in cmd)}")
        if args.dry_run:
            continue
        log_path = os.path.join(out_dir, exp.tag + ".log")
        t0 = time.time()
        with open(log_path, "w") as log:
            rc = subprocess.run(cmd, cwd=ROOT, stdout=log, stderr=subprocess.STDOUT).returncode
        parsed = parse_log(open(log_path).read()) if rc == 0 else None
        summary.append({"tag": exp.tag, "gpus": exp.gpus, "rc": rc, "wall_s": time.time() - t0, **(parsed or {})})
        print(f"   rc={rc} " + (json.dumps(parsed) if parsed else "(no step lines)"))
        time.sleep(3)  # let sockets of the previous job drain
    if summary:
        with open(os.path.join(out_dir, "summary.json"), "w") as f:
            json.dump(summary, f, indent=2)
        print(f"\n{'experiment':<40}{'GPUs':>5}{'tok/s':>12}{'MFU %':>8}{'mem GB':>8}{'s/step':>8}")
        for r in summary:
            if "tokens_per_sec" in r:
                print(f"{r['tag']:<40}{r['gpus']:>5}{r['tokens_per_sec']:>12,.0f}{r['mfu_pct']:>8.1f}"
                      f"{r['peak_mem_gb']:>8.1f}{r['step_time_s']:>8.2f}")
            else:
                print(f"{r['tag']:<40}{r['gpus']:>5}   failed (rc={r['rc']})")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
