"""The five-phase gate and its negative controls on real GPUs (one process per GPU over NVLink).
Skipped on machines with fewer than two GPUs; the single-GPU form is tests/test_allreduce_emulated_gpu.py."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc, extra, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "fp4_all_reduce_b200.harness.gate_dist"] + extra
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    recs = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{") and '"kind": "check"' in l]
    return p.returncode, recs, p.stdout[-3000:] + p.stderr[-3000:]


def _world_sizes():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4, 8) if w <= n]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gate_passes(world):
    if world not in _world_sizes():
        pytest.skip(f"needs {world} GPUs")
    rc, recs, log = _run(world, ["--rows", "1024,333", "--inputs", "bf16,nvfp4", "--epilogues", "0,1", "--reps", "20",
                                 "--graph-calls", "5", "--graph-reps", "5", "--skew-reps", "4"], 29611 + world)
    assert rc == 0, log
    assert len(recs) == 8 and all(r["pass"] for r in recs), recs


@pytest.mark.parametrize("negctl", ["stale", "flip"])
def test_negative_controls_fail_every_cell(negctl):
    rc, recs, log = _run(2, ["--rows", "512", "--reps", "6", "--graph-calls", "3", "--graph-reps", "2", "--skew-reps", "2",
                             "--negctl", negctl], 29631)
    assert rc != 0, log        # every rank exits with 3; the launcher reports that as a failure
    assert recs and all(not r["pass"] for r in recs), recs


def _run_module(nproc, module, extra, port, timeout=900):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", f"fp4_all_reduce_b200.harness.{module}"] + extra
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    recs = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    return p.returncode, recs, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.parametrize("world", [2, 4])
def test_fused_gemm_push_allreduce_matches_host_model(world):
    """Row-parallel GEMM whose epilogue pushes NVFP4 partials into the peers' windows, then the AllReduce kernel in
    pushed-input mode with the norm epilogue: bit for bit against the host model fed with every rank's NVFP4 partial."""
    if world not in _world_sizes():
        pytest.skip(f"needs {world} GPUs")
    rc, recs, log = _run_module(world, "gemm_ar_bench", ["--ms", "512", "--check", "--iters", "2", "--warmup", "1", "--graph", "2"],
                                29651 + world)
    assert rc == 0, log
    checks = [r for r in recs if r.get("kind") == "check"]
    assert len(checks) == 1 and checks[0]["mismatches_vs_host_model"] == 0 and checks[0]["gemm_status"] == 0, checks
    assert all(r.get("status", "ok") == "ok" for r in recs if r.get("kind") == "timing"), recs


def test_comparison_variants_match_host_model_on_two_gpus():
    if 2 not in _world_sizes():
        pytest.skip("needs 2 GPUs")
    rc, recs, log = _run_module(2, "compare_bench", ["--rows", "777", "--check", "--iters", "2", "--warmup", "1", "--graph", "3"], 29661)
    assert rc == 0, log
    checks = [r for r in recs if r.get("kind") == "check"]
    assert len(checks) == 8 and all(r["pass"] for r in checks), checks
