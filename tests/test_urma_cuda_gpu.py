"""URMA over GPU memory (cuda_ipc provider): one-sided write / read between device segments, system-scope atomics and
two-sided send / receive into posted device buffers, within one process on one GPU. The cross-process path (CUDA IPC
handles) is covered by the multi-GPU test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_cuda_ipc_write_read_atomics():
    from umdk_b200 import urma
    a, b = urma.Context("cuda0"), urma.Context("cuda0")
    try:
        ea, eb = a.endpoint(depth=64), b.endpoint(depth=64)
        mem_b = torch.zeros(1 << 18, dtype=torch.float32, device="cuda")
        cnt_b = torch.zeros(16, dtype=torch.int64, device="cuda")
        seg_b = b.register(mem_b, token=21)
        cseg_b = b.register(cnt_b, token=22)
        peer_b = a.import_endpoint(eb.blob)
        rseg, rcnt = a.import_segment(seg_b.blob, token=21), a.import_segment(cseg_b.blob, token=22)
        src = torch.randn(4096, device="cuda")
        ea.write(peer_b, rseg, rseg.va + 4096 * 4, src.data_ptr(), src.numel() * 4)
        ea.wait(1)
        assert torch.equal(mem_b[4096:8192], src)
        back = torch.zeros(4096, device="cuda")
        ea.read(peer_b, rseg, rseg.va + 4096 * 4, back.data_ptr(), back.numel() * 4)
        ea.wait(1)
        assert torch.equal(back, src)
        res = ctypes.c_uint64(0)
        for i in range(100):
            ea.atomic(peer_b, urma.OPC_FADD, rcnt, rcnt.va, 3, 0, ctypes.addressof(res))
        got = ea.wait(100, timeout_ms=10000)
        assert len(got) == 100 and int(cnt_b[0]) == 300 and res.value == 297
        assert ea.compare_swap(peer_b, rcnt, rcnt.va + 8, 0, 77) == 0 and int(cnt_b[1]) == 77
        # wrong token: refused with an error completion, memory untouched
        bad = a.import_segment(seg_b.blob, token=999)
        ea.write(peer_b, bad, bad.va, src.data_ptr(), 16)
        c = ea.wait(1, check=False)
        assert c[0].status == urma.CR_REM_ACCESS_ABORT
    finally:
        a.close()
        b.close()


def test_cuda_ipc_send_recv_into_posted_device_buffers():
    from umdk_b200 import urma
    a, b = urma.Context("cuda0"), urma.Context("cuda0")
    try:
        ea, eb = a.endpoint(depth=64), b.endpoint(depth=64)
        peer_b = a.import_endpoint(eb.blob)
        bufs = [torch.zeros(1024, dtype=torch.float32, device="cuda") for _ in range(3)]
        for i, t in enumerate(bufs):
            eb.post_recv(t, user_ctx=100 + i)
        m0 = torch.randn(1024, device="cuda")
        m1 = torch.randn(256, device="cuda")
        ea.send(peer_b, m0.data_ptr(), m0.numel() * 4, user_ctx=1)
        ea.send(peer_b, m1.data_ptr(), m1.numel() * 4, user_ctx=2, imm=0xABCD)
        sent = ea.wait(2)
        assert [c.user_ctx for c in sent] == [1, 2]
        got = eb.wait(2)
        assert [c.user_ctx for c in got] == [100, 101] and [c.length for c in got] == [4096, 1024]
        assert all(c.flags & urma.CR_FLAG_RECV for c in got) and got[1].imm == 0xABCD
        assert torch.equal(bufs[0], m0) and torch.equal(bufs[1][:256], m1)
        # a message longer than the posted buffer: both sides get an error completion, the buffer is spent
        big = torch.randn(2048, device="cuda")
        ea.send(peer_b, big.data_ptr(), big.numel() * 4, user_ctx=3)
        assert ea.wait(1, check=False)[0].status != urma.CR_SUCCESS
        r = eb.wait(1, check=False)
        assert r[0].status != urma.CR_SUCCESS and r[0].user_ctx == 102
        ea.recover()
        # nothing posted: receiver-not-ready on the sender, nothing arrives
        ea.send(peer_b, m1.data_ptr(), 64, user_ctx=4)
        assert ea.wait(1, check=False)[0].status == urma.CR_RNR
        assert eb.poll() == []
    finally:
        a.close()
        b.close()


@pytest.mark.parametrize("op", ["write", "read", "send"])
def test_urma_perftest_on_gpu_memory(tmp_path, op):
    """The command-line tool with its buffers in GPU memory (`--dev cuda0`), the second endpoint on another GPU when
    the box has one: one-sided verbs and two-sided SEND into posted device buffers."""
    import os
    import subprocess
    from umdk_b200 import _native
    tool = _native.lib_dir() / "bin" / "urma_perftest"
    args = [str(tool), "--dev", "cuda0", "--op", op, "--size", "65536", "--iters", "400", "--depth", "16"]
    if torch.cuda.device_count() >= 2:
        args += ["--peer-dev", "cuda1"]
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"))
    (tmp_path / "urma").mkdir(exist_ok=True)
    p = subprocess.run(args, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=180)
    assert p.returncode == 0 and "urma_perftest: OK" in p.stdout and "errors 0" in p.stdout, p.stdout[-2000:]
    assert f"{op} dev=cuda0 size=65536" in p.stdout


def test_urma_perftest_between_two_gpus_uses_the_direct_path(tmp_path):
    """Two endpoints of one process on two GPUs: the copy must go over NVLink (the devices are given access to each
    other when a segment or a receive buffer of the other GPU is first used; staged through host memory the same copy
    reaches a few tens of GB/s), and an atomic on the other GPU's memory must work."""
    import os
    import re
    import subprocess
    from umdk_b200 import _native
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    tool = _native.lib_dir() / "bin" / "urma_perftest"
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"))
    (tmp_path / "urma").mkdir(exist_ok=True)
    for op, size in (("write", 67108864), ("send", 67108864), ("faa", 8)):
        args = [str(tool), "--dev", "cuda0", "--peer-dev", "cuda1", "--op", op, "--size", str(size), "--iters", "100"]
        p = subprocess.run(args, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=180)
        assert p.returncode == 0 and "urma_perftest: OK" in p.stdout and "errors 0" in p.stdout, p.stdout[-2000:]
        if op != "faa":
            mbs = float(re.search(r"ops/s, ([0-9.]+) MB/s", p.stdout).group(1))
            assert mbs > 200e3, p.stdout   # 64 MiB copies: NVLink gives about 700 GB/s, the host path about 36 GB/s


@pytest.mark.parametrize("op", ["write", "read", "faa"])
def test_bond_device_over_gpu_paths(tmp_path, op):
    """The multipath device with GPU paths (`BOND_DEVICES=cuda0,cuda0`: two contexts, two streams on the GPU) and
    buffers in GPU memory: one-sided operations and atomics go through the bond layer's scheduling, store and
    completion handling untouched by it (two-sided sends of the bond layer use host bounce buffers and stay on host
    devices)."""
    import os
    import subprocess
    from umdk_b200 import _native
    tool = _native.lib_dir() / "bin" / "urma_perftest"
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"), BOND_DEVICES="cuda0,cuda0")
    (tmp_path / "urma").mkdir(exist_ok=True)
    args = [str(tool), "--dev", "bond0", "--mem", "cuda0", "--op", op, "--size", "65536", "--iters", "400"]
    p = subprocess.run(args, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=180)
    assert p.returncode == 0 and "urma_perftest: OK" in p.stdout and "errors 0" in p.stdout, p.stdout[-2000:]
