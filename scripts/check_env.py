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
import subprocess
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


# --------------------------------------------------------------------------- requirement tags
REQUIREMENT_TAGS = ("gpu", "slurm", "multi-node", "wandb", "hf", "gh")
CLUSTER_FILE = ROOT / "configs" / "cluster" / "local.toml"


def load_cluster_config(path: str | os.PathLike | None = None) -> dict:
    """``configs/cluster/local.toml`` (or ``path``) as a dict; empty when the file does not exist."""
    import tomllib

    target = Path(path) if path else CLUSTER_FILE
    if not target.exists():
        return {}
    with open(target, "rb") as fh:
        return tomllib.load(fh)


def parse_requires(text: str | None) -> list[str]:
    """``"gpu, slurm"`` -> ["gpu", "slurm"]; unknown tags are kept and reported as misses."""
    return [t.strip() for t in (text or "").split(",") if t.strip() and t.strip() != "baseline"]


def _result(status: str, message: str, fix: str = "") -> dict:
    return {"status": status, "message": message, "fix": fix}


def require_gpu(cluster: dict) -> dict:
    smi = shutil.which("nvidia-smi")
    if smi:
        try:
            out = subprocess.run([smi, "-L"], capture_output=True, text=True, timeout=20)
            n = len([ln for ln in out.stdout.splitlines() if ln.startswith("GPU ")])
            if out.returncode == 0 and n:
                return _result("ok", f"{n} GPU(s) listed by nvidia-smi")
        except (OSError, subprocess.SubprocessError):
            pass
    nodes = sorted(Path("/dev").glob("nvidia[0-9]*"))
    if nodes:
        return _result("ok", f"{len(nodes)} GPU device node(s) under /dev")
    return _result("miss", "no GPU visible", "run on a GPU node (salloc / srun --gres=gpu:...)")


def require_slurm(cluster: dict) -> dict:
    if not shutil.which("sbatch"):
        return _result("miss", "sbatch not found", "load the SLURM module or run on a login node")
    sl = cluster.get("slurm", {})
    account = sl.get("account") or os.environ.get("SLURM_ACCOUNT", "")
    qos = sl.get("qos") or os.environ.get("SLURM_QOS", "")
    if sl.get("require_account", True) and not account:
        return _result("miss", "no SLURM account configured", "set [slurm].account in configs/cluster/local.toml or $SLURM_ACCOUNT")
    if sl.get("require_qos", False) and not qos:
        return _result("miss", "this cluster requires a QoS and none is configured", "set [slurm].qos or $SLURM_QOS")
    extras = f", qos={qos}" if qos else ""
    return _result("ok", f"sbatch found, account={account or '-'}{extras}")


def require_multi_node(cluster: dict) -> dict:
    if not cluster:
        return _result("miss", "no cluster configuration", "python scripts/check_env.py --init")
    shared = cluster.get("network", {}).get("shared_fs_root", "")
    if not shared:
        return _result("miss", "[network].shared_fs_root is not set", "point it at a filesystem every node mounts")
    root = Path(shared)
    if not root.is_dir():
        return _result("miss", f"shared_fs_root {shared} does not exist on this machine")
    if root.resolve() not in (ROOT.resolve(), *ROOT.resolve().parents):
        return _result("miss", f"the repository ({ROOT}) is not under shared_fs_root ({shared})", "check it out on the shared filesystem")
    ckpt = cluster.get("paths", {}).get("checkpoints_root", "")
    if ckpt and root.resolve() not in (Path(ckpt).resolve(), *Path(ckpt).resolve().parents):
        return _result("miss", f"checkpoints_root ({ckpt}) is not under shared_fs_root ({shared})")
    return _result("warn", "paths are consistent; filesystem type and InfiniBand are not verified from here")


def require_wandb(cluster: dict) -> dict:
    if os.environ.get("WANDB_API_KEY"):
        return _result("ok", "WANDB_API_KEY is set (not validated)")
    return _result("miss", "WANDB_API_KEY is not set", "export WANDB_API_KEY=... or `wandb login`")


def require_hf(cluster: dict) -> dict:
    for var in ("HF_TOKEN", "HUGGING_FACE_HUB_TOKEN"):
        if os.environ.get(var):
            return _result("ok", f"{var} is set")
    return _result("miss", "no Hugging Face token in the environment", "export HF_TOKEN=... or `huggingface-cli login`")


def require_gh(cluster: dict) -> dict:
    gh = shutil.which("gh")
    if not gh:
        return _result("miss", "gh (GitHub CLI) not found", "install it from https://cli.github.com")
    try:
        rc = subprocess.run([gh, "auth", "status"], capture_output=True, text=True, timeout=30).returncode
    except (OSError, subprocess.SubprocessError):
        rc = 1
    return _result("ok", "gh is authenticated") if rc == 0 else _result("miss", "gh is not authenticated", "gh auth login")


_REQUIRE = {"gpu": require_gpu, "slurm": require_slurm, "multi-node": require_multi_node, "wandb": require_wandb,
            "hf": require_hf, "gh": require_gh}


def run_requirements(tags: list[str], cluster: dict) -> dict[str, dict]:
    out = {}
    for tag in tags:
        fn = _REQUIRE.get(tag)
        out[tag] = fn(cluster) if fn else _result("miss", f"unknown requirement tag {tag!r}", f"known: {', '.join(REQUIREMENT_TAGS)}")
    return out


def format_requirements(results: dict[str, dict]) -> str:
    width = max((len(k) for k in results), default=0)
    lines = []
    for tag, r in results.items():
        lines.append(f"[{r['status'].upper():4s}] {tag:<{width}s}  {r['message']}")
        if r["status"] == "miss" and r.get("fix"):
            lines.append(" " * (8 + width) + f"fix: {r['fix']}")
    return "\n".join(lines)


def write_cluster_config(args, force: bool = False) -> Path:
    """``configs/cluster/local.toml`` in the launch scripts' schema, from flags with environment fall-backs."""
    env = os.environ
    target = Path(args.cluster_config) if args.cluster_config else CLUSTER_FILE
    if target.exists() and not force:
        raise FileExistsError(f"{target} exists; pass --force to overwrite")
    scheduler = args.scheduler or ("slurm" if shutil.which("sbatch") else "none")

    def pick(flag, var, default=""):
        return flag if flag not in (None, "") else env.get(var, default)

    def boolean(v, default):
        return default if v is None else str(v).lower() in ("1", "true", "yes")

    body = f"""# written by scripts/check_env.py --init
[cluster]
name = "{pick(args.cluster_name, 'SLURM_CLUSTER_NAME', 'local')}"
scheduler = "{scheduler}"

[slurm]
account = "{pick(args.slurm_account, 'SLURM_ACCOUNT')}"
partition = "{pick(args.slurm_partition, 'SLURM_PARTITION')}"
qos = "{pick(args.slurm_qos, 'SLURM_QOS')}"
default_time = "{args.slurm_time or '01:00:00'}"
default_nodes = {int(args.slurm_nodes or 1)}
default_gpus_per_node = {int(args.slurm_gpus_per_node or 8)}
require_account = {str(boolean(args.require_account, True)).lower()}
require_qos = {str(boolean(args.require_qos, False)).lower()}

[network]
ib_interface = "{args.ib_interface or 'auto'}"
shared_fs_root = "{args.shared_fs_root or ''}"

[paths]
checkpoints_root = "{args.checkpoints_root or ''}"

[credentials]
wandb_entity = "{pick(args.wandb_entity, 'WANDB_ENTITY')}"
hf_user = "{args.hf_user or ''}"
"""
    target.parent.mkdir(parents=True, exist_ok=True)
    target.write_text(body)
    return target


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="check_env")
    ap.add_argument("--requires", default=None, help="comma-separated tags: " + ",".join(REQUIREMENT_TAGS))
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--init", action="store_true", help="write configs/cluster/local.toml")
    ap.add_argument("--non-interactive", action="store_true", help="with --init: take every field from flags / environment")
    ap.add_argument("--force", action="store_true", help="with --init: overwrite an existing file")
    ap.add_argument("--checkpoint-dir", default=None)
    for flag in ("cluster-name", "scheduler", "slurm-account", "slurm-partition", "slurm-qos", "slurm-time", "slurm-nodes",
                 "slurm-gpus-per-node", "require-account", "require-qos", "ib-interface", "shared-fs-root",
                 "checkpoints-root", "wandb-entity", "hf-user", "cluster-config"):
        ap.add_argument(f"--{flag}", default=None)
    args = ap.parse_args(argv)
    if args.non_interactive and not args.init:
        ap.error("--non-interactive only makes sense with --init")
    report = {"python": check_python(), "torch": check_torch(), "layout": check_layout(), "native": check_native(),
              "gpus": check_gpus(), "slurm": check_slurm(), "optional": check_optional(),
              "filesystem": check_filesystem(args.checkpoint_dir)}
    if args.init:
        if not args.non_interactive and sys.stdin.isatty():
            for field, prompt in (("slurm_account", "SLURM account"), ("slurm_partition", "SLURM partition"),
                                  ("shared_fs_root", "shared filesystem root (multi-node)"),
                                  ("checkpoints_root", "checkpoint root")):
                if getattr(args, field) in (None, ""):
                    setattr(args, field, input(f"{prompt} [{getattr(args, field) or ''}]: ").strip() or None)
        try:
            report["cluster_file"] = str(write_cluster_config(args, force=args.force))
        except FileExistsError as exc:
            print(str(exc), file=sys.stderr)
            return 1
    tags = parse_requires(args.requires)
    required = run_requirements(tags, load_cluster_config(args.cluster_config)) if tags else {}
    if required:
        report["requires"] = required
    if args.json:
        print(json.dumps(report, indent=2))
    else:
        for section, body in report.items():
            if section == "requires":
                continue
            if isinstance(body, dict):
                print(f"[{_ok(body.get('ok', True)):7s}] {section}: " + ", ".join(f"{k}={v}" for k, v in body.items() if k != "ok"))
            else:
                print(f"[info   ] {section}: {body}")
        if required:
            print(format_requirements(required))
    hard = ("python", "torch", "layout")
    missed = any(r["status"] == "miss" for r in required.values())
    return 0 if all(report[k]["ok"] for k in hard) and not missed else 1


if __name__ == "__main__":
    sys.exit(main())
