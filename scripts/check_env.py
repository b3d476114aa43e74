#!/usr/bin/env python
"""Pre-flight check of the machine a training job is about to use.

    python scripts/check_env.py [--json] [--init]

Reports, section by section: Python / PyTorch / CUDA versions, the native kernel library (built? loadable?),
GPUs (name, memory, compute capability, peer access), the NCCL / gloo back-ends, SLURM context, the repository
layout, optional integrations (Weights & Biases, HuggingFace cache, tensorboard) and — with ``--init`` — writes a
``configs/cluster/local.toml`` describing the machine for the launch scripts.  Nothing here changes any GPU setting.

Same role as the reference's scripts/check_env.py:97-703.
"""

from __future__ import annotations

import argparse
import importlib
import json
import os
import platform
import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _ok(v: bool) -> str:
    return "ok" if v else "MISSING"


def check_python() -> dict:
    return {"python": platform.python_version(), "executable": sys.executable, "ok": sys.version_info >= (3, 11)}


def check_torch() -> dict:
    try:
        import torch

        return {"torch": torch.__version__, "cuda_runtime": torch.version.cuda, "cuda_available": torch.cuda.is_available(),
                "nccl": torch.distributed.is_nccl_available(), "gloo": torch.distributed.is_gloo_available(), "ok": True}
    except Exception as exc:
        return {"ok": False, "error": str(exc)}


def check_native() -> dict:
    from kempnerforge_b200.ops.build import LIB_PATH, sources

    out = {"library": str(LIB_PATH), "built": LIB_PATH.exists(), "nvcc": shutil.which("nvcc") or "", "sources": len(sources())}
    if LIB_PATH.exists():
        try:
            import ctypes

            ctypes.CDLL(str(LIB_PATH))
            out["loadable"] = True
        except OSError as exc:
            out["loadable"] = False
            out["error"] = str(exc)
    out["ok"] = out["built"] and out.get("loadable", False)
    return out


def check_gpus() -> dict:
    import torch

    if not torch.cuda.is_available():
        return {"count": 0, "ok": False}
    gpus = []
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        gpus.append({"index": i, "name": p.name, "memory_gb": round(p.total_memory / 2**30, 1),
                     "capability": f"{p.major}.{p.minor}", "sms": p.multi_processor_count})
    peer = all(torch.cuda.can_device_access_peer(0, j) for j in range(1, len(gpus))) if len(gpus) > 1 else True
    return {"count": len(gpus), "gpus": gpus, "peer_access_from_gpu0": peer,
            "blackwell": all(g["capability"].startswith("10.") for g in gpus), "ok": True}


def check_slurm() -> dict:
    keys = ("SLURM_JOB_ID", "SLURM_JOB_NODELIST", "SLURM_NTASKS", "SLURM_JOB_PARTITION", "SLURM_RESTART_COUNT")
    env = {k: os.environ[k] for k in keys if k in os.environ}
    return {"in_job": "SLURM_JOB_ID" in env, "sbatch": bool(shutil.which("sbatch")), "env": env, "ok": True}


def check_layout() -> dict:
    need = ["kempnerforge_b200", "csrc", "configs", "scripts/train.py", "bench.py", "tests"]
    missing = [p for p in need if not (ROOT / p).exists()]
    return {"root": str(ROOT), "missing": missing, "ok": not missing}


def check_optional() -> dict:
    out = {}
    for mod in ("wandb", "tensorboard", "datasets", "transformers", "safetensors", "av", "lm_eval"):
        try:
            importlib.import_module(mod)
            out[mod] = True
        except Exception:
            out[mod] = False
    out["wandb_api_key"] = bool(os.environ.get("WANDB_API_KEY"))
    out["hf_home"] = os.environ.get("HF_HOME", str(Path.home() / ".cache" / "huggingface"))
    out["ok"] = True
    return out


def check_filesystem(path: str | None) -> dict:
    target = Path(path or os.environ.get("KF_CHECKPOINT_DIR", "checkpoints"))
    probe_dir = target if target.exists() else target.parent if target.parent.exists() else Path(".")
    usage = shutil.disk_usage(probe_dir)
    writable = os.access(probe_dir, os.W_OK)
    return {"checkpoint_dir": str(target), "free_gb": round(usage.free / 2**30, 1), "writable": writable, "ok": writable}


def write_cluster_file(report: dict) -> Path:
    dst = ROOT / "configs" / "cluster" / "local.toml"
    dst.parent.mkdir(parents=True, exist_ok=True)
    g = report["gpus"]
    lines = ["# written by scripts/check_env.py --init; consumed by the launch scripts, not by training",
             "[cluster]", f'scheduler = "{"slurm" if report["slurm"]["sbatch"] else "local"}"',
             f"gpus_per_node = {g.get('count', 0)}",
             f'gpu_name = "{g["gpus"][0]["name"] if g.get("gpus") else ""}"',
             f'partition = "{report["slurm"]["env"].get("SLURM_JOB_PARTITION", "")}"',
             "[paths]", f'checkpoint_dir = "{report["filesystem"]["checkpoint_dir"]}"',
             f'hf_home = "{report["optional"]["hf_home"]}"', ""]
    dst.write_text("\n".join(lines))
    return dst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--init", action="store_true", help="write configs/cluster/local.toml")
    ap.add_argument("--checkpoint-dir", default=None)
    args = ap.parse_args(argv)
    report = {"python": check_python(), "torch": check_torch(), "layout": check_layout(), "native": check_native(),
              "gpus": check_gpus(), "slurm": check_slurm(), "optional": check_optional(),
              "filesystem": check_filesystem(args.checkpoint_dir)}
    if args.init:
        report["cluster_file"] = str(write_cluster_file(report))
    if args.json:
        print(json.dumps(report, indent=2))
    else:
        for section, body in report.items():
            if isinstance(body, dict):
                print(f"[{_ok(body.get('ok', True)):7s}] {section}: " + ", ".join(f"{k}={v}" for k, v in body.items() if k != "ok"))
            else:
                print(f"[info   ] {section}: {body}")
    hard = ("python", "torch", "layout")
    return 0 if all(report[k]["ok"] for k in hard) else 1


if __name__ == "__main__":
    sys.exit(main())
