"""Scheduler context and resume-path discovery.

"Elastic" here means requeue + auto-resume: a preempted job is started again by the cluster
scheduler, finds the newest checkpoint and continues — possibly on a different number of GPUs,
because checkpoints are stored world-size independent.

Parity: kempnerforge/resilience/elastic.py:21-132.
"""

from __future__ import annotations

import logging
import os
import re
from dataclasses import dataclass
from pathlib import Path

log = logging.getLogger(__name__)
_STEP_RE = re.compile(r"^step_(\d+)$")


@dataclass
class SLURMInfo:
    job_id: str | None = None
    job_name: str | None = None
    node_list: str | None = None
    num_nodes: int = 1
    ntasks_per_node: int = 1
    restart_count: int = 0
    array_task_id: str | None = None
    partition: str | None = None

    @property
    def tasks_per_node(self) -> int:
        return self.ntasks_per_node

    @property
    def is_requeued(self) -> bool:
        return self.restart_count > 0


def get_slurm_info() -> SLURMInfo | None:
    env = os.environ
    if "SLURM_JOB_ID" not in env:
        return None

    def _int(key: str, default: int) -> int:
        try:
            return int(env.get(key, default))
        except ValueError:
            return default

    tpn = env.get("SLURM_NTASKS_PER_NODE", env.get("SLURM_TASKS_PER_NODE", "1"))
    m = re.match(r"\d+", tpn)
    return SLURMInfo(
        job_id=env["SLURM_JOB_ID"],
        job_name=env.get("SLURM_JOB_NAME", ""),
        node_list=env.get("SLURM_JOB_NODELIST", ""),
        num_nodes=_int("SLURM_JOB_NUM_NODES", _int("SLURM_NNODES", 1)),
        ntasks_per_node=int(m.group()) if m else 1,
        restart_count=_int("SLURM_RESTART_COUNT", 0),
        array_task_id=env.get("SLURM_ARRAY_TASK_ID"),
        partition=env.get("SLURM_JOB_PARTITION", ""),
    )


def is_slurm_job() -> bool:
    return "SLURM_JOB_ID" in os.environ


def is_slurm_requeue() -> bool:
    try:
        return int(os.environ.get("SLURM_RESTART_COUNT", "0")) > 0
    except ValueError:
        return False


def list_step_dirs(checkpoint_dir: str | Path) -> list[tuple[int, Path]]:
    root = Path(checkpoint_dir)
    if not root.is_dir():
        return []
    found = []
    for child in root.iterdir():
        m = _STEP_RE.match(child.name)
        if m and child.is_dir():
            found.append((int(m.group(1)), child))
    return sorted(found)


def resolve_resume_path(checkpoint_dir: str | Path) -> Path | None:
    """The ``latest`` link when it points at an existing directory, else the highest ``step_N``."""
    root = Path(checkpoint_dir)
    latest = root / "latest"
    if latest.exists():
        target = latest.resolve()
        if target.is_dir():
            return target
    steps = list_step_dirs(root)
    return steps[-1][1] if steps else None


def log_job_info() -> None:
    info = get_slurm_info()
    if info is None:
        log.info("Not running under SLURM")
        return
    log.info("SLURM job %s (%s) nodes=%d tasks/node=%d partition=%s restart_count=%d", info.job_id,
             info.job_name, info.num_nodes, info.tasks_per_node, info.partition, info.restart_count)
    if info.restart_count > 0:
        log.info("Job was requeued (restart #%d): resuming from the newest checkpoint", info.restart_count)
