"""The benchmark harness and the cluster benchmark driver stay runnable (CPU, tiny shapes)."""

import json

import torch

from benchmarks import cluster_bench
from benchmarks.runner import Case, main, run_benchmark


def test_run_benchmark_times_a_case_and_derives_rates():
    calls = []
    res = run_benchmark(Case("toy", lambda: calls.append(1), tokens_per_iter=100, flops_per_iter=1e6), warmup=2,
                        iterations=3, device=torch.device("cpu"))
    assert len(calls) == 5 and res.step_time_ms > 0 and res.tokens_per_sec > 0 and "tflops" in res.extra
    assert "toy" in res.row()


def test_data_suite_runs_and_saves_json(tmp_path):
    out = tmp_path / "bench.json"
    results = main(["--suite", "data", "--warmup", "1", "--iterations", "1", "--output", str(out)])
    assert len(results) >= 3
    saved = json.loads(out.read_text())
    assert saved["results"][0]["name"].startswith("MemoryMappedDataset")


def test_cluster_driver_matrices_and_log_parsing():
    assert {"mfu_scaling", "moe_ep", "moe_packed"} <= set(cluster_bench.MATRICES)
    exp = cluster_bench.MATRICES["mfu_scaling"][2]
    cmd = cluster_bench.launch_command(exp, steps=5, port=29999, extra="--data.pin_memory=false")
    assert "--distributed.tp=2" in cmd and "--train.max_steps=5" in cmd and "--nproc-per-node=2" in cmd
    big = [e for e in cluster_bench.MATRICES["mfu_scaling"] if e.gpus > 8][0]
    assert cluster_bench.launch_command(big, 5, 29999, "") is None  # no SLURM allocation here
    log = ("noise\n[step 5] loss=2.5 | lr=3.00e-04 | grad_norm=0.8 | tok/s=10,000 | mfu=40.0% | mem=10.0/180GB | step_time=0.50s\n"
           "[step 10] loss=2.4 | lr=3.00e-04 | grad_norm=0.7 | tok/s=12,000 | mfu=44.0% | mem=11.0/180GB | step_time=0.40s\n")
    parsed = cluster_bench.parse_log(log, skip=1)
    assert parsed["tokens_per_sec"] == 12000 and parsed["peak_mem_gb"] == 11.0 and parsed["last_step"] == 10
