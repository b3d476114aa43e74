"""Multi-GPU behaviour (NCCL over NVLink): launched as child processes, one rank per GPU."""

import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import json, os, sys, torch
sys.path.insert(0, os.environ["KF_ROOT"])
from kempnerforge_b200.config import config_from_dict
from kempnerforge_b200.training.trainer import Trainer
world = int(os.environ["WORLD_SIZE"]); rank = int(os.environ["RANK"])
cfg = config_from_dict({
    "model": dict(dim=512, n_layers=4, n_heads=8, n_kv_heads=2, vocab_size=4096, ffn_hidden_dim=1536, max_seq_len=256),
    "train": dict(batch_size=2, seq_len=256, max_steps=10, mixed_precision="bf16", activation_checkpointing="full", seed=0),
    "optimizer": dict(lr=1e-3, name=os.environ.get("KF_TEST_OPTIMIZER") or "adamw"), "scheduler": dict(warmup_steps=0, name="constant"),
    "distributed": dict(dp_shard=world, param_sharding=os.environ.get("KF_TEST_PARAM_SHARDING") or "resident"),
    "metrics": dict(log_interval=1000)})
emulate = int(os.environ.get("KF_TEST_EMULATE_RANKS") or 0)   # one process stepping on the batches of that many ranks
if emulate:
    cfg.train.grad_accum_steps = emulate
t = Trainer(cfg, transport=os.environ.get("KF_TRANSPORT") or None)
gens = [torch.Generator().manual_seed(100 + r) for r in (range(emulate) if emulate else [rank])]
out = []
for step in range(4):
    micro = []
    for g in gens:
        tok = torch.randint(0, 4096, (2, 257), generator=g)
        micro.append({"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()})
    out.append(t.train_step(micro))
if t.engine is not None:
    t.engine.wait_all()
def whole(p):
    g = getattr(p, "_kf_flat", None)
    return t.engine.full_parameter(p) if g is not None and getattr(g, "sharded", False) else p.detach()
flat = torch.cat([whole(p).float().flatten() for p in t.model.parameters()])
mem = t.engine.memory_report() if hasattr(t.engine, "memory_report") else {}
digest = torch.stack([flat.sum(), flat.abs().sum(), flat.pow(2).sum()])
gathered = [torch.zeros_like(digest) for _ in range(world)]
if world > 1:
    torch.distributed.all_gather(gathered, digest)
else:
    gathered = [digest]
if rank == 0:
    same = all(torch.equal(gathered[0], x) for x in gathered)
    print("RESULT " + json.dumps({"losses": [o["loss"] for o in out], "norms": [o["grad_norm"] for o in out], "replicas_identical": same,
                                  "digest": [float(x) for x in digest], "engine": type(t.engine).__name__, "mem": mem,
                                  "status": __import__("kempnerforge_b200.ops.cuda", fromlist=["x"]).read_status()}))
if torch.distributed.is_initialized():
    torch.distributed.destroy_process_group()
'''


def _run(world: int, transport: str = "", multimem: bool = True, tmp_dir: str = "/tmp", sharding: str = "resident",
         optimizer: str = "", emulate: int = 0):
    script = os.path.join(tmp_dir, f"kf_multi_gpu_worker_{os.getpid()}.py")
    with open(script, "w") as f:
        f.write(WORKER)
    env = dict(os.environ, KF_ROOT=ROOT, NCCL_NVLS_ENABLE="0", KF_TRANSPORT=transport,
               KF_SYMM_MULTIMEM="1" if multimem else "0", KF_TEST_PARAM_SHARDING=sharding, KF_TEST_OPTIMIZER=optimizer,
               KF_TEST_EMULATE_RANKS=str(emulate) if emulate else "")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29631", script]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, (res.stdout[-1500:] + "\n" + res.stderr[-4000:])
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_sharded_data_parallel_two_gpus():
    r = _run(2, transport="collective")
    assert r["replicas_identical"], "ranks ended with different parameters"
    assert all(l == l and 0 < l < 20 for l in r["losses"]) and all(n > 0 for n in r["norms"])
    assert r["losses"][-1] < r["losses"][0] + 0.5


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("multimem", [False, True])
def test_symmetric_transport_matches_collectives(multimem):
    """Fused reduce-scatter / AdamW / publish kernels over peer memory against the NCCL path."""
    base = _run(2, transport="collective")
    fused = _run(2, transport="symmetric", multimem=multimem)
    assert fused["replicas_identical"]
    for a, b in zip(base["losses"], fused["losses"]):
        assert abs(a - b) < 5e-2, (base["losses"], fused["losses"])
    for a, b in zip(base["norms"], fused["norms"]):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (base["norms"], fused["norms"])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("transport", ["symmetric", "collective"])
def test_sharded_parameters_match_resident_parameters(transport):
    """ZeRO-3 (weights gathered inside the GEMMs that read them, gradients reduce-scattered into shards) against the
    resident engine on the same data: same losses, gradient norms and final parameters."""
    base = _run(2, transport="collective")
    z3 = _run(2, transport=transport, multimem=False, sharding="sharded")
    assert z3["engine"] == "ShardedDataParallelEngine" and z3["status"] == 0
    for a, b in zip(base["losses"], z3["losses"]):
        assert abs(a - b) < 5e-2, (base["losses"], z3["losses"])
    for a, b in zip(base["norms"], z3["norms"]):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (base["norms"], z3["norms"])
    for a, b in zip(base["digest"], z3["digest"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (base["digest"], z3["digest"])
    assert z3["mem"]["param_shards"] > 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("optimizer,transport", [("lion", "collective"), ("muon", "collective"), ("muon", "symmetric")])
def test_whole_parameter_optimizers_under_data_parallelism(optimizer, transport):
    """Lion and Muon step on whole parameters: with two data-parallel ranks every rank must receive the whole averaged
    gradient (NCCL all-reduce, or reduce-scatter + gather over peer memory), so the replicas stay identical and follow
    the run of ONE process that accumulates both ranks' batches.  Muon also divides its Newton-Schulz work."""
    one = _run(1, transport="collective", optimizer=optimizer, emulate=2)
    two = _run(2, transport=transport, multimem=False, optimizer=optimizer)
    assert two["replicas_identical"], "ranks ended with different parameters"
    assert all(x == x for x in one["losses"] + two["losses"])
    # rank 0 reports its own micro-batch's loss; compare what does not depend on the rank: norms and parameters
    for a, b in zip(one["norms"], two["norms"]):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (one["norms"], two["norms"])
    for a, b in zip(one["digest"], two["digest"]):
        assert abs(a - b) < 1e-2 * max(1.0, abs(a)), (one["digest"], two["digest"])


GEMM_RS_WORKER = r'''
import json, os, sys, torch
import torch.distributed as dist
sys.path.insert(0, os.environ["KF_ROOT"])
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
from kempnerforge_b200.comm.fused_tp import GemmRSContext
from kempnerforge_b200.ops import cuda as K
dev = torch.device("cuda")
B, S, D, Kl = 2, 128 * world * 2, 768, 320  # Kl is a multiple of 64 (needed by the (K, D) layout)
T = B * S
ctx = GemmRSContext(dist.group.WORLD, dev, T, D)
errs = []
for call in range(5):
    g = torch.Generator(device="cuda").manual_seed(1000 * call + rank)
    x = torch.randn(T, Kl, device=dev, dtype=torch.bfloat16, generator=g)
    w = torch.randn(D, Kl, device=dev, dtype=torch.bfloat16, generator=g) * 0.05
    res = torch.randn(T // world, D, device=dev, dtype=torch.bfloat16, generator=g) if call % 2 else None
    if call % 2 == 0:
        out = K.gemm_reduce_scatter(x, w, ctx, S, residual=res)
    else:  # the same product with the weight stored (K, D): the layout of the input-gradient GEMM
        out = K.gemm_reduce_scatter(x, w.t().contiguous(), ctx, S, residual=res, w_kn=True)
    full = (x.float() @ w.float().t())
    dist.all_reduce(full)
    mine = full.view(B, world, S // world, D)[:, rank].reshape(T // world, D)
    if res is not None:
        mine = mine + res.float()
    errs.append(((out.float() - mine).abs().max() / mine.abs().max()).item())
torch.cuda.synchronize()
status = K.read_status()
worst = torch.tensor([max(errs), float(status)], device=dev)
dist.all_reduce(worst, op=dist.ReduceOp.MAX)
if rank == 0:
    print("RESULT " + json.dumps({"max_rel_err": worst[0].item(), "status": worst[1].item()}))
dist.destroy_process_group()
'''


def _run_script(script_text: str, world: int, name: str, extra_env: dict | None = None):
    path = os.path.join("/tmp", f"kf_{name}_{os.getpid()}.py")
    with open(path, "w") as f:
        f.write(script_text)
    env = dict(os.environ, KF_ROOT=ROOT, NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29641", path]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, (res.stdout[-1500:] + "\n" + res.stderr[-4000:])
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def _worlds():
    """World sizes to test on this box: 2, and 4 / 8 when that many GPUs are visible (owner rotation, shard
    arithmetic and flag layouts differ with the number of ranks)."""
    n = torch.cuda.device_count()
    return [w for w in (2, 4, 8) if w <= n] or [2]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("world", _worlds())
def test_fused_gemm_reduce_scatter_matches_nccl(world):
    """GEMM whose epilogue pushes tiles to the owning rank and reduces them, against matmul + all-reduce."""
    r = _run_script(GEMM_RS_WORKER, world, "gemm_rs")
    assert r["status"] == 0
    assert r["max_rel_err"] < 2e-2, r


AG_GEMM_WORKER = r'''
import json, os, sys, torch
import torch.distributed as dist
sys.path.insert(0, os.environ["KF_ROOT"])
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
from kempnerforge_b200.comm.fused_tp import AgGemmContext
from kempnerforge_b200.ops import cuda as K
dev = torch.device("cuda")
B, S, N, Kd = 2, 128 * world * 2, 520, 384
T = B * S
ctx = AgGemmContext(dist.group.WORLD, dev, T, Kd)
errs = []
for call in range(5):
    g = torch.Generator(device="cuda").manual_seed(1000 * call + rank)
    xs = torch.randn(T // world, Kd, device=dev, dtype=torch.bfloat16, generator=g)
    w = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16, generator=g) * 0.05
    if call % 2 == 0:
        out = K.all_gather_gemm(xs, w, ctx, S)
    else:
        out = K.all_gather_gemm(xs, w.t().contiguous(), ctx, S, w_kn=True)
    parts = [torch.empty_like(xs) for _ in range(world)]
    dist.all_gather(parts, xs)
    full = torch.stack([p.view(B, S // world, Kd) for p in parts], dim=1).reshape(T, Kd)
    want = full.float() @ w.float().t()
    errs.append(((out.float() - want).abs().max() / want.abs().max()).item())
torch.cuda.synchronize()
worst = torch.tensor([max(errs), float(K.read_status())], device=dev)
dist.all_reduce(worst, op=dist.ReduceOp.MAX)
if rank == 0:
    print("RESULT " + json.dumps({"max_rel_err": worst[0].item(), "status": worst[1].item()}))
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("world", _worlds())
def test_fused_all_gather_gemm_matches_nccl(world):
    """GEMM whose copy warps push the local shard to the peers, against all-gather + matmul."""
    r = _run_script(AG_GEMM_WORKER, world, "ag_gemm")
    assert r["status"] == 0
    assert r["max_rel_err"] < 2e-2, r


_DIST = '"distributed": dict(dp_shard=world,'
assert _DIST in WORKER
TP_WORKER = WORKER.replace(_DIST, '"distributed": dict(tp=world, dp_shard=1,') \
                  .replace("g = torch.Generator().manual_seed(100 + rank)", "g = torch.Generator().manual_seed(100)")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tensor_parallel_fused_kernels_match_library_collectives():
    """TP=2 with sequence parallelism: all-gather+GEMM / GEMM+reduce-scatter kernels against NCCL collectives."""
    assert "tp=world" in TP_WORKER
    fused = _run_script(TP_WORKER, 2, "tp_fused", {"KF_TP_FUSED": "1", "KF_TRANSPORT": ""})
    plain = _run_script(TP_WORKER, 2, "tp_plain", {"KF_TP_FUSED": "0", "KF_TRANSPORT": ""})
    for a, b in zip(plain["losses"], fused["losses"]):
        assert abs(a - b) < 5e-2, (plain["losses"], fused["losses"])
    for a, b in zip(plain["norms"], fused["norms"]):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (plain["norms"], fused["norms"])


EP_WORKER = WORKER.replace(
    "model\": dict(dim=512, n_layers=4, n_heads=8, n_kv_heads=2, vocab_size=4096, ffn_hidden_dim=1536, max_seq_len=256)",
    "model\": dict(dim=512, n_layers=2, n_heads=8, n_kv_heads=2, vocab_size=4096, ffn_hidden_dim=1024, max_seq_len=256, "
    "num_experts=8, moe_top_k=2, moe_packed_experts=True, moe_aux_loss_weight=0.01)") \
    .replace(_DIST, '"distributed": dict(ep=world, ep_in_dp=True, dp_shard=world,')


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("world", _worlds())
def test_expert_parallel_peer_memory_dispatch_matches_all_to_all(world):
    """Experts sharded over the data-parallel ranks (EP = 2, 4 or 8 of 8 experts): rows exchanged by our peer-store
    kernels against NCCL all-to-all."""
    assert "num_experts=8" in EP_WORKER and "ep_in_dp=True" in EP_WORKER
    fused = _run_script(EP_WORKER, world, "ep_fused", {"KF_EP_FUSED": "1", "KF_TRANSPORT": "collective"})
    plain = _run_script(EP_WORKER, world, "ep_plain", {"KF_EP_FUSED": "0", "KF_TRANSPORT": "collective"})
    for a, b in zip(plain["losses"], fused["losses"]):
        assert abs(a - b) < 5e-2, (plain["losses"], fused["losses"])
    for a, b in zip(plain["norms"], fused["norms"]):
        assert abs(a - b) < 8e-2 * max(1.0, abs(a)), (plain["norms"], fused["norms"])
