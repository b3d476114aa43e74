"""Process-environment helpers of the distributed set-up: rank discovery, InfiniBand interface detection,
NCCL defaults, rendezvous address, mesh shapes.  Mirrors tests/unit/test_distributed.py of the reference
(environment part); everything is faked on the host."""

from __future__ import annotations

import subprocess
from types import SimpleNamespace

import pytest

from kempnerforge_b200.config.sections import DistributedConfig
from kempnerforge_b200.parallel import setup as kf_setup

_RANK_VARS = ("RANK", "LOCAL_RANK", "WORLD_SIZE", "SLURM_PROCID", "SLURM_LOCALID", "SLURM_NTASKS")


_ENV_VARS = _RANK_VARS + ("NCCL_SOCKET_IFNAME", "GLOO_SOCKET_IFNAME", "NCCL_IB_DISABLE", "NCCL_NET_GDR_LEVEL",
                          "TORCH_NCCL_ASYNC_ERROR_HANDLING", "MASTER_ADDR", "MASTER_PORT", "SLURM_JOB_NODELIST", "SLURM_JOB_ID")


@pytest.fixture
def clean_env(monkeypatch):
    import os

    saved = {k: os.environ.get(k) for k in _ENV_VARS}
    for k in _ENV_VARS:
        os.environ.pop(k, None)
    yield monkeypatch
    monkeypatch.undo()
    for k, v in saved.items():        # the functions under test export variables themselves: put the process back
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


def test_world_info_precedence(clean_env):
    import os

    assert kf_setup.get_world_info() == (0, 0, 1)
    assert (os.environ["RANK"], os.environ["LOCAL_RANK"], os.environ["WORLD_SIZE"]) == ("0", "0", "1")   # exported for env://
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        del os.environ[k]
    clean_env.setenv("SLURM_PROCID", "5")
    clean_env.setenv("SLURM_LOCALID", "1")
    clean_env.setenv("SLURM_NTASKS", "8")
    assert kf_setup.get_world_info() == (5, 1, 8)
    assert (os.environ["RANK"], os.environ["LOCAL_RANK"], os.environ["WORLD_SIZE"]) == ("5", "1", "8")
    clean_env.setenv("RANK", "3")
    clean_env.setenv("LOCAL_RANK", "3")
    clean_env.setenv("WORLD_SIZE", "4")
    assert kf_setup.get_world_info() == (3, 3, 4)      # torchrun variables win over SLURM


def _fake_ip(monkeypatch, stdout=None, error=None):
    def run(cmd, **kw):
        if error:
            raise error
        return SimpleNamespace(stdout=stdout, returncode=0)

    monkeypatch.setattr(subprocess, "run", run)


@pytest.mark.parametrize("stdout,want", [
    ("lo UNKNOWN 127.0.0.1/8\neth0 UP 10.0.0.2/24\nib0 UP 10.1.0.2/16\n", "ib0"),
    ("ib1 DOWN\nib2 UP 10.1.0.2/16\nib3 UP 10.1.0.3/16\n", "ib2"),
    ("lo UNKNOWN 127.0.0.1/8\neth0 UP 10.0.0.2/24\n", None),
    ("ib0 DOWN 10.1.0.2/16\n", None),
    ("", None),
])
def test_ib_interface_detection(clean_env, stdout, want):
    _fake_ip(clean_env, stdout)
    assert kf_setup._detect_ib_interface() == want


def test_ib_detection_survives_a_missing_tool(clean_env):
    _fake_ip(clean_env, error=FileNotFoundError("ip"))
    assert kf_setup._detect_ib_interface() is None
    _fake_ip(clean_env, error=subprocess.TimeoutExpired("ip", 5))
    assert kf_setup._detect_ib_interface() is None


def test_nccl_defaults_follow_the_detected_interface(clean_env):
    import os

    _fake_ip(clean_env, "ib0 UP 10.1.0.2/16\n")
    kf_setup._set_nccl_env()
    assert os.environ["NCCL_SOCKET_IFNAME"] == "ib0" and os.environ["GLOO_SOCKET_IFNAME"] == "ib0"
    assert os.environ["NCCL_IB_DISABLE"] == "0" and os.environ["TORCH_NCCL_ASYNC_ERROR_HANDLING"] == "1"


def test_nccl_defaults_never_override_the_user(clean_env):
    import os

    clean_env.setenv("NCCL_SOCKET_IFNAME", "eth7")
    clean_env.setenv("GLOO_SOCKET_IFNAME", "eth7")
    clean_env.setenv("TORCH_NCCL_ASYNC_ERROR_HANDLING", "0")
    _fake_ip(clean_env, "ib0 UP 10.1.0.2/16\n")
    kf_setup._set_nccl_env()
    assert os.environ["NCCL_SOCKET_IFNAME"] == "eth7" and os.environ["TORCH_NCCL_ASYNC_ERROR_HANDLING"] == "0"
    assert os.environ["NCCL_IB_DISABLE"] == "0"            # a default nobody set: filled in


def test_nccl_defaults_without_infiniband(clean_env):
    import os

    _fake_ip(clean_env, "eth0 UP 10.0.0.2/24\n")
    kf_setup._set_nccl_env()
    assert "NCCL_SOCKET_IFNAME" not in os.environ and "GLOO_SOCKET_IFNAME" not in os.environ
    assert os.environ["TORCH_NCCL_ASYNC_ERROR_HANDLING"] == "1" and os.environ["NCCL_IB_DISABLE"] == "0"


def test_gloo_follows_the_interface_the_user_named_for_nccl_and_a_disabled_watchdog_is_warned_about(clean_env, caplog):
    import os

    clean_env.setenv("NCCL_SOCKET_IFNAME", "eth3")
    clean_env.setenv("TORCH_NCCL_ASYNC_ERROR_HANDLING", "0")
    _fake_ip(clean_env, error=AssertionError("no detection when the user named an interface"))
    with caplog.at_level("WARNING", logger=kf_setup.log.name):
        kf_setup._set_nccl_env()
    assert os.environ["GLOO_SOCKET_IFNAME"] == "eth3" and os.environ["TORCH_NCCL_ASYNC_ERROR_HANDLING"] == "0"
    assert any("TORCH_NCCL_ASYNC_ERROR_HANDLING=0" in r.getMessage() for r in caplog.records)


def test_master_resolution(clean_env):
    import os

    kf_setup._resolve_master()
    assert os.environ["MASTER_ADDR"] == "127.0.0.1" and 1024 < int(os.environ["MASTER_PORT"]) < 65536
    clean_env.delenv("MASTER_ADDR")
    clean_env.delenv("MASTER_PORT")
    clean_env.setenv("SLURM_JOB_NODELIST", "node[01-04]")
    clean_env.setenv("SLURM_JOB_ID", "4242")
    clean_env.setattr(subprocess, "run", lambda cmd, **kw: SimpleNamespace(stdout="node01\nnode02\n"))
    kf_setup._resolve_master()
    first_port = os.environ["MASTER_PORT"]
    assert os.environ["MASTER_ADDR"] == "node01" and 20000 <= int(first_port) <= 60000
    clean_env.delenv("MASTER_PORT")
    kf_setup._resolve_master()
    assert os.environ["MASTER_PORT"] == first_port      # every rank of a job derives the same port
    clean_env.setenv("MASTER_ADDR", "10.9.9.9")
    kf_setup._resolve_master()
    assert os.environ["MASTER_ADDR"] == "10.9.9.9"


@pytest.mark.parametrize("kw,world,sizes,names", [
    (dict(), 8, (8,), ("dp_shard",)),
    (dict(tp=2), 8, (4, 2), ("dp_shard", "tp")),
    (dict(tp=8), 8, (1, 8), ("dp_shard", "tp")),
    (dict(pp=2, tp=2), 8, (2, 2, 2), ("pp", "dp_shard", "tp")),
    (dict(dp_replicate=2, dp_shard=4), 8, (2, 4), ("dp_replicate", "dp_shard")),
    (dict(ep=2), 8, (4, 2), ("dp_shard", "ep")),
    (dict(ep=8, ep_in_dp=True), 8, (8,), ("dp_shard",)),
    (dict(), 1, (1,), ("dp_shard",)),
])
def test_mesh_shapes(kw, world, sizes, names):
    assert kf_setup.mesh_shape(DistributedConfig(**kw), world) == (sizes, names)


def test_mesh_shape_rejects_a_world_the_factors_do_not_divide():
    with pytest.raises(ValueError):
        kf_setup.mesh_shape(DistributedConfig(tp=3), 8)
    with pytest.raises(ValueError):
        kf_setup.mesh_shape(DistributedConfig(dp_shard=3, tp=2), 8)
