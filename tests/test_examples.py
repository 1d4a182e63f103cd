"""The example programs run as a user would start them (CPU: gloo, one and two processes) and, on a GPU, the
low-latency sample against its small-ops pipeline."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EX = os.path.join(ROOT, "examples")


def _run(cmd, timeout=300, env_extra=None):
    env = dict(os.environ)
    env["CUDA_VISIBLE_DEVICES"] = env.get("CUDA_VISIBLE_DEVICES", "") if env_extra is None else env_extra.get(
        "CUDA_VISIBLE_DEVICES", env.get("CUDA_VISIBLE_DEVICES", ""))
    p = subprocess.run(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=timeout)
    return p.returncode, p.stdout


def _json_lines(out):
    return [json.loads(l) for l in out.splitlines() if l.startswith("{")]


def test_prefill_sample_single_process_cpu():
    rc, out = _run([sys.executable, os.path.join(EX, "moe_dispatch_combine_prefill_sample.py"), "--tokens", "64",
                    "--hidden", "256", "--experts-per-rank", "8", "--topk", "2"],
                   env_extra={"CUDA_VISIBLE_DEVICES": ""})
    assert rc == 0, out[-3000:]
    assert _json_lines(out)[0]["ok"] is True


def test_prefill_sample_two_processes_gloo():
    rc, out = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                    "--master-addr", "127.0.0.1", "--master-port", "29541",
                    os.path.join(EX, "moe_dispatch_combine_prefill_sample.py"), "--tokens", "48", "--hidden", "256",
                    "--experts-per-rank", "4", "--topk", "2", "--no-fp8"], env_extra={"CUDA_VISIBLE_DEVICES": ""})
    assert rc == 0, out[-3000:]
    assert _json_lines(out)[0]["ok"] is True


def test_diagnose_matrix_flags_slow_rank():
    sys.path.insert(0, EX)
    try:
        from utils import diagnose_matrix
    finally:
        sys.path.pop(0)
    m = torch.full((8, 8), 10.0)
    m[:, 3] = 100.0       # everybody waits long for rank 3
    m[5, 6] = 300.0       # one bad pair
    d = diagnose_matrix(m)
    assert d["abnormal_cols"] == [3] and d["abnormal_rows"] == [] and (5, 6) in d["abnormal_points"]


@pytest.mark.gpu
def test_fused_deep_moe_sample_gpu():
    rc, out = _run([sys.executable, os.path.join(EX, "fused_deep_moe_sample.py"), "--tokens", "64", "--hidden",
                    "1024", "--ffn", "512", "--experts", "16", "--topk", "4", "--iters", "3", "--warmup", "1"])
    assert rc == 0, out[-3000:]
    assert _json_lines(out)[0]["ok"] is True


@pytest.mark.gpu
def test_prefill_sample_gpu():
    rc, out = _run([sys.executable, os.path.join(EX, "moe_dispatch_combine_prefill_sample.py"), "--tokens", "256",
                    "--hidden", "1024", "--experts-per-rank", "8", "--topk", "4", "--iters", "3", "--warmup", "1"])
    assert rc == 0, out[-3000:]
    assert _json_lines(out)[0]["ok"] is True


@pytest.mark.parametrize("script,args", [
    ("urma_sample.py", ["--self"]),
    ("urpc_echo.py", ["--calls", "50", "--psk", "ab" * 32]),
    ("umq_pingpong.py", ["--rounds", "50"]),
    ("urpc_live_queues.py", ["--calls", "40"]),
    ("umq_sub_queues.py", ["--connections", "16"]),
    ("dlock_counter.py", ["--threads", "3", "--increments", "50", "--fair"]),
])
def test_host_library_samples(script, args, tmp_path):
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"))
    (tmp_path / "urma").mkdir()
    p = subprocess.run([sys.executable, os.path.join(EX, script)] + args, cwd=ROOT, env=env, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=120)
    assert p.returncode == 0, p.stdout[-2000:]
    assert _json_lines(p.stdout)[-1]["ok"] is True
