"""Host libraries under AddressSanitizer / LeakSanitizer and ThreadSanitizer: the sanitizer flavours are built into
build/lib_<kind>/ and the UMQ and URPC tools run their self-tests there without a single report. (The reference
ships asan / tsan build configurations for the same purpose; kernels have no such tool on this hardware pool and are
covered by bounds checks and oracles instead.)"""
import os
import shutil
import subprocess

import pytest

from umdk_b200 import _build


def _run(exe, args, tmp_path, extra_env=None):
    env = dict(os.environ, URMA_SHM_DIR=str(tmp_path / "urma"))
    env.update(extra_env or {})
    (tmp_path / "urma").mkdir(exist_ok=True)
    p = subprocess.run([str(exe), *args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=400,
                       env=env)
    return p.returncode, p.stdout


needs_gxx = pytest.mark.skipif(not os.path.exists("/usr/bin/g++") and shutil.which("g++") is None,
                               reason="no host compiler")


@needs_gxx
def test_address_and_leak_sanitizer_clean(tmp_path):
    outs = _build.build_sanitized("address", only=_build.HOST_LIBS + (
        "tool_umq_perftest", "tool_urpc_perftest", "tool_urma_perftest", "tool_urma_raw_sample", "tool_dlock_example"))
    rc, out = _run(outs["tool_umq_perftest"], ["--iters", "500", "--flow-control"], tmp_path)
    assert rc == 0 and "umq_perftest: OK" in out and "Sanitizer" not in out, out[-3000:]
    # self-test flavour: huge buffers, sub queues over the jetty pool, a pulled large message
    rc, out = _run(outs["tool_umq_perftest"], ["--iters", "300", "--selftest"], tmp_path)
    assert rc == 0 and "umq_perftest: OK" in out and "Sanitizer" not in out, out[-3000:]
    # (includes a queue pair joining and leaving the attached channel through the control-plane task engine)
    rc, out = _run(outs["tool_urpc_perftest"], ["--selftest", "--iters", "300"], tmp_path)
    assert rc == 0 and "urpc_perftest: OK" in out and "Sanitizer" not in out, out[-3000:]
    rc, out = _run(outs["tool_urpc_perftest"], ["--iters", "600", "--queues", "3"], tmp_path)   # three queue pairs
    assert rc == 0 and "urpc_perftest: OK" in out and "Sanitizer" not in out, out[-3000:]
    # the shared-memory device itself: four threads of mixed traffic (rings of requests, the table of requests in
    # flight, messages reassembled in the posted buffers), the raw-API walk-through, and the lock service
    rc, out = _run(outs["tool_urma_perftest"], ["--stress", "4", "--iters", "500", "--size", "4096"], tmp_path)
    assert rc == 0 and "all data verified" in out and "Sanitizer" not in out, out[-3000:]
    rc, out = _run(outs["tool_urma_raw_sample"], [], tmp_path)
    assert rc == 0 and "urma_raw_sample: OK" in out and "Sanitizer" not in out, out[-3000:]
    rc, out = _run(outs["tool_dlock_example"], ["--selftest", "--iters", "500"], tmp_path)
    assert rc == 0 and "dlock_example: OK" in out and "Sanitizer" not in out, out[-3000:]


@needs_gxx
def test_thread_sanitizer_clean(tmp_path):
    outs = _build.build_sanitized("thread", only=_build.HOST_LIBS + ("tool_umq_perftest", "tool_urpc_perftest",
                                                                      "tool_ums_perftest", "tool_urma_perftest",
                                                                      "tool_dlock_example"))
    # the shared-memory device with four threads at once: sends of one slot and of several fragments, writes, reads
    # and atomics, executed by the contexts' own threads and by the polling threads themselves (and by the contexts'
    # threads alone)
    rc, out = _run(outs["tool_urma_perftest"], ["--stress", "4", "--iters", "400", "--size", "4096"], tmp_path)
    assert rc == 0 and "all data verified" in out and "ThreadSanitizer" not in out, out[-3000:]
    rc, out = _run(outs["tool_urma_perftest"], ["--stress", "3", "--iters", "300", "--size", "1000"], tmp_path,
                   {"URMA_SHM_INLINE_POLL": "0"})
    assert rc == 0 and "all data verified" in out and "ThreadSanitizer" not in out, out[-3000:]
    for _ in range(2):   # the teardown race this guards against showed up in about one run out of three
        rc, out = _run(outs["tool_umq_perftest"], ["--iters", "300", "--flow-control"], tmp_path)
        assert rc == 0 and "umq_perftest: OK" in out and "ThreadSanitizer" not in out, out[-3000:]
    rc, out = _run(outs["tool_urpc_perftest"], ["--iters", "300", "--queues", "3"], tmp_path)
    assert rc == 0 and "urpc_perftest: OK" in out and "ThreadSanitizer" not in out, out[-3000:]
    # control-plane task engine against the polling server thread and the client: queue add / remove on a live channel
    rc, out = _run(outs["tool_urpc_perftest"], ["--selftest", "--iters", "200"], tmp_path)
    assert rc == 0 and "urpc_perftest: OK" in out and "ThreadSanitizer" not in out, out[-3000:]
    rc, out = _run(outs["tool_umq_perftest"], ["--iters", "200", "--selftest"], tmp_path)
    assert rc == 0 and "umq_perftest: OK" in out and "ThreadSanitizer" not in out, out[-3000:]
    # stream sockets: link groups (40 connections, echo threads, control rings, link reaping) and the fallback paths
    ums_env = {"UMS_SHM_DIR": str(tmp_path / "ums"), "UMS_LINK_LINGER_MS": "100"}
    rc, out = _run(outs["tool_ums_perftest"], ["--linkgroups"], tmp_path, ums_env)
    assert rc == 0 and ": OK" in out and "ThreadSanitizer" not in out, out[-3000:]
    rc, out = _run(outs["tool_ums_perftest"], ["--selftest", "--iters", "300"], tmp_path, ums_env)
    assert rc == 0 and "ums_perftest: OK" in out and "ThreadSanitizer" not in out, out[-3000:]
    # several connections at once: every thread keeps its own view of the connection table
    rc, out = _run(outs["tool_ums_perftest"], ["--conns", "4", "--iters", "300"], tmp_path, ums_env)
    assert rc == 0 and "ums_perftest: OK" in out and "ThreadSanitizer" not in out, out[-3000:]
    # lock service: three clients in parallel against the command thread, then the self-test with its restart
    rc, out = _run(outs["tool_dlock_example"], ["--clients", "3", "--iters", "300"], tmp_path)
    assert rc == 0 and "dlock_example: OK" in out and "ThreadSanitizer" not in out, out[-3000:]
