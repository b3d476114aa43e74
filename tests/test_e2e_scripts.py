"""End-to-end runs of the command-line entry points in child processes (CPU): train -> checkpoint -> eval /
generate, SIGTERM -> emergency checkpoint -> automatic resume.  Mirrors the reference's smoke pipelines
(tests/smoke/test_smoke.py) at toy size."""

import json
import os
import signal
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = ["--model.dim=64", "--model.n_layers=2", "--model.n_heads=4", "--model.n_kv_heads=2", "--model.vocab_size=256",
        "--model.max_seq_len=64", "--train.batch_size=2", "--train.seq_len=32", "--train.mixed_precision=fp32",
        "--train.compile_model=false", "--metrics.log_interval=1", "--optimizer.lr=1e-3", "--scheduler.warmup_steps=0",
        "--metrics.enable_wandb=false", "--metrics.enable_tensorboard=false"]


def _env():
    return dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1")


def _train(args, **kw):
    cmd = [sys.executable, os.path.join(ROOT, "scripts", "train.py"), os.path.join(ROOT, "configs", "train", "debug.toml"),
           *TINY, *args]
    return subprocess.run(cmd, capture_output=True, text=True, env=_env(), timeout=600, cwd=ROOT, **kw)


def _steps_logged(text: str) -> list[int]:
    import re

    return [int(m) for m in re.findall(r"\[step (\d+)\]", text)]


def test_train_checkpoint_eval_generate_pipeline(tmp_path):
    ckpt = str(tmp_path / "ckpt")
    r = _train([f"--checkpoint.dir={ckpt}", "--checkpoint.interval=4", "--train.max_steps=8"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    out = r.stdout + r.stderr
    assert 8 in _steps_logged(out)
    assert os.path.isdir(os.path.join(ckpt, "step_8")) and os.path.exists(os.path.join(ckpt, "latest"))
    meta = json.load(open(os.path.join(ckpt, "step_8", "metadata.json")))
    assert meta["step"] == 8
    # resume: two more steps continue from step 8, not from 0
    r2 = _train([f"--checkpoint.dir={ckpt}", "--checkpoint.interval=100", "--train.max_steps=10"])
    assert r2.returncode == 0, r2.stdout[-2000:] + r2.stderr[-2000:]
    steps = _steps_logged(r2.stdout + r2.stderr)
    assert steps and min(steps) >= 9 and max(steps) == 10, steps
    # the evaluation script reads the same checkpoint and a small token shard
    import numpy as np

    data_dir = tmp_path / "eval_tokens"
    data_dir.mkdir()
    np.save(data_dir / "shard_0.npy", np.random.default_rng(0).integers(0, 256, size=4096, dtype=np.uint16))
    ev = subprocess.run([sys.executable, os.path.join(ROOT, "scripts", "eval.py"),
                         os.path.join(ROOT, "configs", "train", "debug.toml"), *TINY, f"--checkpoint.load_path={ckpt}/latest",
                         f"--eval.dataset_path={data_dir}", "--eval.steps=2"],
                        capture_output=True, text=True, env=_env(), timeout=600, cwd=ROOT)
    assert ev.returncode == 0, ev.stdout[-2000:] + ev.stderr[-2000:]
    assert "loss" in (ev.stdout + ev.stderr).lower()


def test_sigterm_writes_emergency_checkpoint_and_resumes(tmp_path):
    ckpt = str(tmp_path / "ckpt")
    cmd = [sys.executable, os.path.join(ROOT, "scripts", "train.py"), os.path.join(ROOT, "configs", "train", "debug.toml"),
           *TINY, f"--checkpoint.dir={ckpt}", "--checkpoint.interval=100000", "--train.max_steps=100000"]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=_env(), cwd=ROOT)
    seen = ""
    deadline = time.time() + 300
    try:
        while time.time() < deadline:  # wait until the loop is really running
            line = proc.stdout.readline()
            if not line:
                break
            seen += line
            if "[step 3]" in line:
                break
        assert "[step 3]" in seen, seen[-3000:]
        proc.send_signal(signal.SIGTERM)
        rest, _ = proc.communicate(timeout=300)
        seen += rest
    finally:
        if proc.poll() is None:
            proc.kill()
    assert proc.returncode == 0, seen[-3000:]
    assert "emergency checkpoint" in seen
    saved = sorted(d for d in os.listdir(ckpt) if d.startswith("step_"))
    assert saved, os.listdir(ckpt)
    last_step = int(saved[-1].split("_")[1])
    assert last_step >= 3 and os.path.exists(os.path.join(ckpt, "latest"))
    r = _train([f"--checkpoint.dir={ckpt}", "--checkpoint.interval=100000", f"--train.max_steps={last_step + 2}"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    steps = _steps_logged(r.stdout + r.stderr)
    assert steps and min(steps) == last_step + 1, (last_step, steps)


def test_sigmoid_moe_with_full_activation_checkpointing_trains(tmp_path):
    """DeepSeek-style routing (bias balancing, shared expert, first layer dense) under full recomputation: the
    recomputed blocks must route exactly as their first pass did, or the run stops with a shape mismatch."""
    r = _train([f"--checkpoint.dir={tmp_path / 'ck'}", "--checkpoint.interval=1000", "--train.max_steps=6",
                "--model.num_experts=4", "--model.moe_top_k=2", "--model.moe_router=sigmoid_topk",
                "--model.moe_shared_experts=1", "--model.moe_first_k_dense=1", "--model.moe_router_z_loss_weight=0.001",
                "--train.activation_checkpointing=full"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert 6 in _steps_logged(r.stdout + r.stderr)


def _torchrun(nproc, args, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "scripts", "train.py"),
           os.path.join(ROOT, "configs", "train", "debug.toml"), *TINY, *args]
    env = _env()
    env.pop("MASTER_ADDR", None)
    return subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=300, cwd=ROOT)


_MOE = ["--model.num_experts=4", "--model.moe_top_k=2"]


@pytest.mark.parametrize("dims", [
    ["--distributed.dp_shard=2"],
    ["--distributed.tp=2", "--distributed.dp_shard=1"],
    ["--distributed.pp=2", "--distributed.dp_shard=1", "--train.grad_accum_steps=2"],
    ["--distributed.ep=2", "--distributed.dp_shard=1", *_MOE],
    ["--distributed.ep=2", "--distributed.ep_in_dp=true", "--distributed.dp_shard=2", *_MOE, "--model.moe_packed_experts=true"],
    ["--distributed.dp_shard=2", "--optimizer.name=muon"],
    ["--distributed.dp_shard=2", "--train.mixed_precision=fp8", "--train.activation_checkpointing=full"],
], ids=["dp2", "tp2", "pp2", "ep2", "ep2_in_dp", "dp2_muon", "dp2_fp8"])
def test_two_rank_runs_through_the_launcher_and_resume(tmp_path, dims):
    """`torchrun scripts/train.py` on two gloo ranks for every parallel mode: trains, writes one checkpoint that both
    ranks contribute to, and a second launch resumes from it."""
    ckpt = str(tmp_path / "ckpt")
    port = 29800 + (hash(tuple(dims)) % 100)
    r = _torchrun(2, [f"--checkpoint.dir={ckpt}", "--checkpoint.interval=3", "--train.max_steps=3", *dims], port)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert 3 in _steps_logged(r.stdout + r.stderr)
    assert os.path.isdir(os.path.join(ckpt, "step_3"))
    r2 = _torchrun(2, [f"--checkpoint.dir={ckpt}", "--checkpoint.interval=100", "--train.max_steps=5", *dims], port + 1)
    assert r2.returncode == 0, r2.stdout[-2000:] + r2.stderr[-3000:]
    steps = _steps_logged(r2.stdout + r2.stderr)
    assert steps and min(steps) >= 4 and max(steps) == 5, steps
    if any(d.startswith("--distributed.pp=") for d in dims):
        # every stage wrote a complete sub-checkpoint; the converter merges them into one model
        step_dir = os.path.join(ckpt, "step_5")
        for stage in ("pp0", "pp1"):
            assert os.path.exists(os.path.join(step_dir, stage, ".metadata"))
            assert os.path.exists(os.path.join(step_dir, stage, "train_state.pt"))
        cfg = tmp_path / "model.toml"
        cfg.write_text("[model]\ndim = 64\nn_layers = 2\nn_heads = 4\nn_kv_heads = 2\nvocab_size = 256\nmax_seq_len = 64\n")
        conv = subprocess.run([sys.executable, os.path.join(ROOT, "scripts", "convert_checkpoint.py"), "--config", str(cfg),
                               "to-hf", step_dir, str(tmp_path / "hf")], capture_output=True, text=True, env=_env(),
                              timeout=300, cwd=ROOT)
        assert conv.returncode == 0, conv.stderr[-2000:]
        from safetensors.torch import load_file

        names = set(load_file(str(tmp_path / "hf" / "model.safetensors")))
        assert {"model.embed_tokens.weight", "lm_head.weight", "model.layers.0.mlp.down_proj.weight",
                "model.layers.1.mlp.down_proj.weight"} <= names


@pytest.mark.parametrize("opts", [
    ["--optimizer.name=schedule_free_adamw", "--scheduler.name=none"],
    ["--checkpoint.async_mode=async"],
    ["--train.mixed_precision=bf16", "--train.activation_checkpointing=selective"],
    ["--optimizer.name=lion", "--train.grad_accum_steps=2", "--scheduler.name=wsd", "--scheduler.stable_steps=2"],
], ids=["schedule_free", "async_ckpt", "bf16_selective_ac", "lion_accum_wsd"])
def test_single_process_variants_train_and_resume(tmp_path, opts):
    ckpt = str(tmp_path / "ckpt")
    r = _train([f"--checkpoint.dir={ckpt}", "--checkpoint.interval=3", "--train.max_steps=3", *opts])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert os.path.isdir(os.path.join(ckpt, "step_3")) and os.path.exists(os.path.join(ckpt, "latest"))
    r2 = _train([f"--checkpoint.dir={ckpt}", "--checkpoint.interval=100", "--train.max_steps=5", *opts])
    assert r2.returncode == 0, r2.stdout[-2000:] + r2.stderr[-3000:]
    steps = _steps_logged(r2.stdout + r2.stderr)
    assert steps and min(steps) >= 4 and max(steps) == 5, steps



def test_mixture_with_a_training_phase_through_the_training_script(tmp_path):
    """Two token sources mixed 3:1, an annealing phase at step 3 that flips the weights and halves the LR."""
    import numpy as np

    rng = np.random.default_rng(0)
    for name in ("web", "code"):
        d = tmp_path / name
        d.mkdir()
        np.save(d / "shard.npy", rng.integers(0, 256, size=33 * 40, dtype=np.uint16))
    cfg = tmp_path / "mix.toml"
    cfg.write_text(f"""
[[data.datasets]]
path = "{tmp_path / 'web'}"
name = "web"
weight = 3.0
[[data.datasets]]
path = "{tmp_path / 'code'}"
name = "code"
weight = 1.0
[[data.phases]]
start_step = 3
lr_scale = 0.5
dataset_weights = {{ web = 1.0, code = 3.0 }}
""")
    cmd = [sys.executable, os.path.join(ROOT, "scripts", "train.py"), str(cfg), *TINY, "--train.max_steps=5",
           "--data.num_workers=0", f"--checkpoint.dir={tmp_path / 'ck'}", "--checkpoint.interval=1000",
           "--scheduler.name=constant"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=_env(), timeout=300, cwd=ROOT)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert 5 in _steps_logged(out) and "Entering data phase 0 at step 3" in out
    import re

    lrs = {int(s): float(v) for s, v in re.findall(r"\[step (\d+)\].*?lr=([0-9.e+-]+)", out)}
    assert lrs[2] == pytest.approx(1e-3) and lrs[5] == pytest.approx(5e-4)
    # per-source metrics on the logged steps: a loss near ln(vocab) and a token count for every source that was drawn
    per_source = re.findall(r"\[step (\d+)\] (?=.*loss/)(.*)", out)
    assert per_source, out[-2000:]
    seen = set()
    for _, line in per_source:
        for name, value in re.findall(r"loss/(\w+)=([0-9.]+)", line):
            seen.add(name)
            assert 3.0 < float(value) < 8.0
        assert re.search(r"data/(web|code)/tokens=", line)
    assert seen == {"web", "code"}


def test_the_evaluation_script_refuses_to_run_without_a_checkpoint(tmp_path):
    """A mistyped ``--checkpoint.load_path`` must not end in metrics of freshly initialised weights."""
    import numpy as np

    data_dir = tmp_path / "eval_tokens"
    data_dir.mkdir()
    np.save(data_dir / "shard_0.npy", np.random.default_rng(0).integers(0, 256, size=2048, dtype=np.uint16))
    ev = subprocess.run([sys.executable, os.path.join(ROOT, "scripts", "eval.py"),
                         os.path.join(ROOT, "configs", "train", "debug.toml"), *TINY,
                         f"--checkpoint.load_path={tmp_path / 'no_such_run' / 'step_10'}",
                         f"--eval.dataset_path={data_dir}", "--eval.steps=1"],
                        capture_output=True, text=True, env=_env(), timeout=600, cwd=ROOT)
    assert ev.returncode == 1, ev.stdout[-1000:] + ev.stderr[-1000:]
    assert "no checkpoint found" in ev.stderr and "eval/loss" not in ev.stdout
