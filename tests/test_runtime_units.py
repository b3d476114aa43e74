"""Collective deadlines with a fake work handle, seeding rules, memory-map lifetime, GPU health probe on CPU,
environment checker.

Mirrors tests/unit/test_collective_timeouts.py, test_distributed_seed.py, test_dataset_mmap_cleanup.py and
test_check_env.py of the reference (failures are produced on the host: a fake of the failing call).
"""

from __future__ import annotations

import importlib.util
import random
import sys
from datetime import timedelta
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist

from kempnerforge_b200.data.dataset import MemoryMappedDataset
from kempnerforge_b200.parallel import setup as kf_setup
from kempnerforge_b200.resilience import health

ROOT = Path(__file__).resolve().parents[1]


class _Work:
    def __init__(self, result=True, raises=None):
        self.result, self.raises, self.seen = result, raises, None

    def wait(self, timeout=None):
        self.seen = timeout
        if self.raises:
            raise self.raises
        return self.result


def _fake_group(monkeypatch, work, world=2):
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: world)
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "gloo")

    def all_reduce(t, group=None, async_op=False):
        t.fill_(world)
        return work

    monkeypatch.setattr(dist, "all_reduce", all_reduce)
    monkeypatch.setattr(dist, "barrier", lambda group=None, async_op=False: work)


# --------------------------------------------------------------------------- deadlines
def test_health_check_passes_the_deadline_to_wait(monkeypatch):
    w = _Work(True)
    _fake_group(monkeypatch, w)
    assert health.check_nccl_health(timeout_sec=2.5) is True
    assert w.seen == timedelta(seconds=2.5)


def test_health_check_false_when_wait_times_out_or_raises(monkeypatch):
    _fake_group(monkeypatch, _Work(False))
    assert health.check_nccl_health(timeout_sec=0.1) is False
    _fake_group(monkeypatch, _Work(raises=RuntimeError("peer went away")))
    assert health.check_nccl_health(timeout_sec=0.1) is False


def test_health_check_false_on_a_wrong_sum(monkeypatch):
    w = _Work(True)
    _fake_group(monkeypatch, w, world=2)
    monkeypatch.setattr(dist, "all_reduce", lambda t, group=None, async_op=False: (t.fill_(1.0), w)[1])
    assert health.check_nccl_health(timeout_sec=0.1) is False


def test_health_check_true_without_a_process_group(monkeypatch):
    monkeypatch.setattr(dist, "is_initialized", lambda: False)
    assert health.check_nccl_health() is True


def test_barrier_with_timeout_raises_with_the_reason(monkeypatch):
    w = _Work(False)
    _fake_group(monkeypatch, w)
    with pytest.raises(RuntimeError, match="timed out after 0.25"):
        kf_setup.barrier_with_timeout(0.25)
    assert w.seen == timedelta(seconds=0.25)
    _fake_group(monkeypatch, _Work(True))
    kf_setup.barrier_with_timeout(0.25)  # returns normally


def test_gpu_health_probe_never_raises_on_cpu(monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    out = health.check_gpu_health()
    assert out["healthy"] is False and "CUDA" in out["error"]
    assert health.check_native_kernel_status() == 0


# --------------------------------------------------------------------------- seeding
def _draws():
    return random.random(), float(np.random.rand()), float(torch.rand(1))


def test_set_seed_covers_python_numpy_and_torch():
    kf_setup.set_seed(123)
    a = _draws()
    kf_setup.set_seed(123)
    assert _draws() == a
    kf_setup.set_seed(124)
    b = _draws()
    assert all(x != y for x, y in zip(a, b))


def test_set_seed_differs_per_pipeline_stage_only():
    kf_setup.set_seed(7, pp_rank=0)
    a = _draws()
    kf_setup.set_seed(7, pp_rank=1)
    b = _draws()
    assert a != b
    kf_setup.set_seed(8, pp_rank=0)  # seed + pp_rank is what counts
    assert _draws() == b


# --------------------------------------------------------------------------- memory maps
def _write_shards(d: Path, n=3, tokens=64):
    for i in range(n):
        np.save(d / f"s{i}.npy", np.arange(tokens, dtype=np.uint16) + i)


def test_mmap_dataset_close_is_idempotent(tmp_path):
    _write_shards(tmp_path)
    ds = MemoryMappedDataset(str(tmp_path), seq_len=16)
    assert len(ds) == 12 and len(ds._mmaps) == 3
    ds.close()
    assert ds._mmaps == []
    ds.close()


def test_mmap_dataset_releases_earlier_maps_when_a_later_file_is_bad(tmp_path, monkeypatch):
    _write_shards(tmp_path)
    opened, closed = [], []
    real_load = np.load

    def load(path, *a, **k):
        if path.endswith("s2.npy"):
            raise OSError("truncated shard")
        arr = real_load(path, *a, **k)
        opened.append(arr)
        return arr

    monkeypatch.setattr(np, "load", load)
    real_close = MemoryMappedDataset.close

    def close(self):
        closed.append(len(self._mmaps))
        real_close(self)

    monkeypatch.setattr(MemoryMappedDataset, "close", close)
    with pytest.raises(OSError, match="truncated"):
        MemoryMappedDataset(str(tmp_path), seq_len=16)
    assert len(opened) == 2 and closed and closed[0] == 2


def test_mmap_dataset_bin_files_and_missing_dir(tmp_path):
    (np.arange(40, dtype=np.uint16)).tofile(tmp_path / "a.bin")       # 80 bytes -> divisible by 4 -> read as uint32
    ds = MemoryMappedDataset(str(tmp_path), seq_len=5, file_pattern="*.bin")
    assert len(ds) == 4
    ds.close()
    with pytest.raises(FileNotFoundError):
        MemoryMappedDataset(str(tmp_path), seq_len=5, file_pattern="*.none")


# --------------------------------------------------------------------------- environment checker
def _check_env():
    spec = importlib.util.spec_from_file_location("kf_check_env", ROOT / "scripts" / "check_env.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["kf_check_env"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_check_env_sections_report_without_a_gpu(tmp_path):
    ce = _check_env()
    for fn in (ce.check_python, ce.check_torch, ce.check_native, ce.check_gpus, ce.check_slurm, ce.check_layout,
               ce.check_optional):
        out = fn()
        assert isinstance(out, dict) and out
    fs = ce.check_filesystem(str(tmp_path))
    assert isinstance(fs, dict)
    assert isinstance(ce.check_filesystem(None), dict)


def test_check_env_main_returns_an_exit_code(capsys):
    ce = _check_env()
    rc = ce.main([])
    out = capsys.readouterr().out
    assert rc in (0, 1) and "python" in out.lower() and "torch" in out.lower()


# --------------------------------------------------------------------------- activation-checkpoint phases
def test_checkpoint_phase_contexts_nest_and_reset():
    from torch.utils.checkpoint import checkpoint

    from kempnerforge_b200.models import recompute

    assert recompute.phase() is None
    fwd, rec = recompute.checkpoint_contexts()
    with fwd:
        assert recompute.phase() == "forward"
        with rec:
            assert recompute.phase() == "recompute"
        assert recompute.phase() == "forward"
    assert recompute.phase() is None
    seen = []

    def body(x):
        seen.append(recompute.phase())
        return x.sin() * x          # saves tensors, so the backward pass has to recompute the region

    x = torch.ones(3, requires_grad=True)
    y = checkpoint(body, x, use_reentrant=False, context_fn=recompute.checkpoint_contexts)
    y.sum().backward()
    assert seen == ["forward", "recompute"] and recompute.phase() is None


def test_side_stream_publication_is_off_without_the_symmetric_transport():
    from kempnerforge_b200.models.transformer import Transformer
    from kempnerforge_b200.config.sections import ModelConfig
    from kempnerforge_b200.parallel.engine import DataParallelEngine

    m = Transformer(ModelConfig(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48, max_seq_len=16))
    eng = DataParallelEngine(m, None, transport="collective")
    assert eng.publish_on_side_stream(eng.groups) is False
    eng.after_optimizer_step()      # single process: nothing to publish, nothing raises
    eng.release()


# --------------------------------------------------------------------------- check_env: requirement tags and --init
def _check_env():
    import importlib.util

    spec = importlib.util.spec_from_file_location("kf_check_env", Path(__file__).resolve().parents[1] / "scripts" / "check_env.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_check_env_requirement_tags(monkeypatch, tmp_path):
    ce = _check_env()
    assert ce.parse_requires(" gpu, slurm ,,hf") == ["gpu", "slurm", "hf"]
    assert ce.parse_requires(None) == []
    monkeypatch.delenv("WANDB_API_KEY", raising=False)
    monkeypatch.delenv("HF_TOKEN", raising=False)
    monkeypatch.delenv("HUGGING_FACE_HUB_TOKEN", raising=False)
    out = ce.run_requirements(["wandb", "hf", "nonsense"], {})
    assert [r["status"] for r in out.values()] == ["miss", "miss", "miss"]
    assert "unknown" in out["nonsense"]["message"]
    monkeypatch.setenv("WANDB_API_KEY", "k")
    monkeypatch.setenv("HUGGING_FACE_HUB_TOKEN", "t")
    out = ce.run_requirements(["wandb", "hf"], {})
    assert [r["status"] for r in out.values()] == ["ok", "ok"]
    text = ce.format_requirements({"hf": {"status": "miss", "message": "no token", "fix": "export HF_TOKEN"}})
    assert "[MISS]" in text and "fix: export HF_TOKEN" in text


def test_check_env_slurm_and_multi_node_rules(monkeypatch, tmp_path):
    ce = _check_env()
    monkeypatch.setattr(ce.shutil, "which", lambda name: None)
    assert ce.require_slurm({})["status"] == "miss"
    monkeypatch.setattr(ce.shutil, "which", lambda name: "/usr/bin/" + name)
    monkeypatch.delenv("SLURM_ACCOUNT", raising=False)
    monkeypatch.delenv("SLURM_QOS", raising=False)
    assert ce.require_slurm({"slurm": {"require_account": True}})["status"] == "miss"
    assert ce.require_slurm({"slurm": {"require_account": False}})["status"] == "ok"
    assert ce.require_slurm({"slurm": {"account": "lab", "require_qos": True}})["status"] == "miss"
    assert ce.require_slurm({"slurm": {"account": "lab", "qos": "high", "require_qos": True}})["status"] == "ok"
    # multi-node: needs a configuration, a shared root that exists, and the repository under it
    assert ce.require_multi_node({})["status"] == "miss"
    assert ce.require_multi_node({"network": {"shared_fs_root": ""}})["status"] == "miss"
    assert ce.require_multi_node({"network": {"shared_fs_root": str(tmp_path / "absent")}})["status"] == "miss"
    assert ce.require_multi_node({"network": {"shared_fs_root": str(tmp_path)}})["status"] == "miss"  # repo elsewhere
    root = str(ce.ROOT.parent)
    assert ce.require_multi_node({"network": {"shared_fs_root": root}})["status"] == "warn"
    cfg = {"network": {"shared_fs_root": root}, "paths": {"checkpoints_root": str(tmp_path)}}
    assert ce.require_multi_node(cfg)["status"] == "miss"
    cfg["paths"]["checkpoints_root"] = str(ce.ROOT / "checkpoints")
    assert ce.require_multi_node(cfg)["status"] == "warn"


def test_check_env_init_writes_the_cluster_schema_and_refuses_to_overwrite(monkeypatch, tmp_path, capsys):
    import tomllib

    ce = _check_env()
    target = tmp_path / "cluster.toml"
    monkeypatch.setenv("SLURM_PARTITION", "gpu_part")
    argv = ["--init", "--non-interactive", "--cluster-config", str(target), "--slurm-account", "lab", "--require-qos", "true",
            "--slurm-nodes", "4", "--shared-fs-root", "/shared", "--wandb-entity", "team"]
    assert ce.main(argv) == 0
    cfg = tomllib.loads(target.read_text())
    assert set(cfg) == {"cluster", "slurm", "network", "paths", "credentials"}
    assert cfg["slurm"]["account"] == "lab" and cfg["slurm"]["partition"] == "gpu_part"
    assert cfg["slurm"]["require_qos"] is True and cfg["slurm"]["require_account"] is True
    assert cfg["slurm"]["default_nodes"] == 4 and cfg["slurm"]["default_gpus_per_node"] == 8
    assert cfg["network"] == {"ib_interface": "auto", "shared_fs_root": "/shared"}
    assert cfg["credentials"]["wandb_entity"] == "team"
    assert ce.load_cluster_config(target) == cfg
    capsys.readouterr()
    assert ce.main(argv) == 1 and "exists" in capsys.readouterr().err
    assert ce.main(argv + ["--force", "--slurm-account", "other"]) == 0
    assert tomllib.loads(target.read_text())["slurm"]["account"] == "other"


def test_check_env_exit_code_follows_required_misses(monkeypatch, capsys):
    import json as _json

    ce = _check_env()
    monkeypatch.delenv("HF_TOKEN", raising=False)
    monkeypatch.delenv("HUGGING_FACE_HUB_TOKEN", raising=False)
    assert ce.main(["--requires", "hf", "--json"]) == 1
    report = _json.loads(capsys.readouterr().out)
    assert report["requires"]["hf"]["status"] == "miss"
    monkeypatch.setenv("HF_TOKEN", "x")
    assert ce.main(["--requires", "hf"]) == 0
    assert "[OK  ] hf" in capsys.readouterr().out
    with pytest.raises(SystemExit):
        ce.main(["--non-interactive"])


def test_codebase_map_is_in_sync_with_the_source():
    """``codebase-map.json`` is generated from the source tree; a stale file fails here."""
    import subprocess
    import sys as _sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([_sys.executable, str(root / "scripts" / "build_codebase_map.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
