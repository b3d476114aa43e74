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


# --------------------------------------------------------------------------- headline benchmark script (host-side parts)
def _bench_module():
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("kf_bench_script", Path(__file__).resolve().parents[1] / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _args(**kw):
    from types import SimpleNamespace

    base = dict(tp=1, ep=1, pp=1, ep_in_dp=False)
    base.update(kw)
    return SimpleNamespace(**base)


def test_bench_mesh_dims_and_labels():
    b = _bench_module()
    assert b.mesh_dims(_args(), 8) == ({"dp_shard": 8}, 8, "dp8")
    assert b.mesh_dims(_args(tp=2), 8) == ({"dp_shard": 4, "tp": 2}, 4, "tp2xdp4")
    assert b.mesh_dims(_args(ep=2), 2) == ({"dp_shard": 1, "ep": 2}, 1, "ep2xdp1")
    assert b.mesh_dims(_args(ep=8, ep_in_dp=True), 8) == ({"ep": 8, "ep_in_dp": True, "dp_shard": 8}, 8, "ep8-in-dp8")
    dims, n, label = b.mesh_dims(_args(pp=2), 8)
    assert dims == {"dp_shard": 4, "pp": 2, "pp_schedule": "1f1b"} and n == 4 and label == "pp2xdp4"
    assert b.mesh_dims(_args(pp=2, tp=2), 8)[2] == "pp2xtp2xdp2"


def test_bench_models_are_the_configured_shapes():
    from kempnerforge_b200.config.sections import DistributedConfig, ModelConfig

    b = _bench_module()
    cfgs = {k: ModelConfig(**v) for k, v in b.MODELS.items()}
    assert abs(cfgs["llama3_8b"].num_params_estimate / 1e9 - 8.03) < 0.05
    assert cfgs["llama_13b"].computed_ffn_hidden_dim == 13824 and cfgs["llama_13b"].n_layers == 40
    fine = cfgs["moe_fine"]
    assert fine.computed_expert_ffn_hidden_dim == 1408 and fine.num_experts == 64 and fine.moe_top_k == 6
    assert [fine.is_moe_layer(i) for i in range(3)] == [False, True, True] and fine.computed_ffn_hidden_dim == 10944
    assert str(fine.moe_router) == "sigmoid_topk" and fine.moe_shared_experts == 2
    top2 = cfgs["moe_8x"]
    assert top2.num_experts == 8 and top2.moe_top_k == 2 and all(top2.is_moe_layer(i) for i in range(24))
    for world, kw in ((8, dict(tp=2)), (8, dict(pp=2)), (8, dict(ep=8, ep_in_dp=True)), (2, dict(ep=2))):
        dims = b.mesh_dims(_args(**kw), world)[0]
        DistributedConfig(**dims).resolve(world)          # every mesh the script can ask for is a valid one
