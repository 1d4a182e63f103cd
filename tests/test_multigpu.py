"""Real multi-GPU runs (one process per GPU, NCCL bootstrap, kernels over NVLink peer memory)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _torchrun(script, nproc, timeout=240):
    env = dict(os.environ)
    env.setdefault("URMA_SHM_DIR", f"/tmp/umdk_urma_test_{os.getpid()}")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(HERE, script)]
    p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)
    return p.returncode, p.stdout


def test_ep_kernels_across_gpus():
    n = min(torch.cuda.device_count(), 8)
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    rc, out = _torchrun("mp_ep_worker.py", n)
    errors = "\n".join(ln for ln in out.splitlines() if "MP_WORKER_ERROR" in ln)
    assert rc == 0 and "MP_EP_OK" in out, errors + "\n" + out[-3000:]


def test_tp_kernels_allreduce_and_urma_across_gpus():
    n = min(torch.cuda.device_count(), 8)
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    rc, out = _torchrun("mp_tp_worker.py", n)
    errors = "\n".join(ln for ln in out.splitlines() if "MP_WORKER_ERROR" in ln)
    assert rc == 0 and "MP_TP_OK" in out, errors + "\n" + out[-3000:]
    # on GPUs that can join an NVLink multicast object the in-switch all-reduce must have run on the package's own
    # multicast heap: a silent fall-back to the peer-pointer algorithms would hide a broken heap
    from umdk_b200 import _native
    line = [ln for ln in out.splitlines() if "MP_TP_OK" in ln][-1]
    print(line)
    if _native.cam().umdk_mc_supported():
        assert "nvls=ok" in line, out[-4000:]


def test_rank_leaves_between_steps_and_survivors_stop_cleanly():
    """Failure handling without a GPU fault: a rank departs between steps, the others learn of it on the host before
    their next launch (NVLS off, plain peer loads)."""
    n = 4 if torch.cuda.device_count() >= 4 else 2
    rc, out = _torchrun("mp_leave_worker.py", n)
    assert rc == 0 and out.count("MP_LEAVE_OK") == n, out[-4000:]
