"""Randomised call sequences against the URMA API on the shared-memory provider (in one process, two contexts),
checked against a byte-array model of the remote segment: whatever the sequence of writes, reads, atomics, bad tokens
and out-of-range addresses, data must match the model, errors must come back as error completions (never a crash) and
nothing may be left in the queues. Plays the role of the reference's libFuzzer harness over its mocked provider
(test/urma/fuzz/urma_api_fuzz.c), with hypothesis generating the sequences."""
import ctypes
import os

import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

SEG_BYTES = 4096

op = st.one_of(
    st.tuples(st.just("write"), st.integers(0, SEG_BYTES - 8), st.integers(1, 512), st.integers(0, 255)),
    st.tuples(st.just("read"), st.integers(0, SEG_BYTES - 8), st.integers(1, 512), st.just(0)),
    st.tuples(st.just("fadd"), st.integers(0, SEG_BYTES // 8 - 1), st.integers(0, 1 << 20), st.just(0)),
    st.tuples(st.just("cas"), st.integers(0, SEG_BYTES // 8 - 1), st.integers(0, 3), st.integers(0, 3)),
    st.tuples(st.just("oob_write"), st.integers(SEG_BYTES - 4, SEG_BYTES + 4096), st.integers(8, 256), st.just(0)),
    st.tuples(st.just("bad_token_write"), st.integers(0, SEG_BYTES - 64), st.integers(1, 64), st.just(0)),
    st.tuples(st.just("ro_write"), st.integers(0, 64), st.integers(1, 32), st.just(0)),
)


@pytest.fixture(scope="module")
def world(tmp_path_factory):
    os.environ.setdefault("URMA_SHM_DIR", str(tmp_path_factory.mktemp("urma_fuzz")))
    from umdk_b200 import urma
    a, b = urma.Context("shm0"), urma.Context("shm0")
    ea, eb = a.endpoint(depth=64, recv_token=3), b.endpoint(depth=64, recv_token=3)
    mem = torch.zeros(SEG_BYTES, dtype=torch.uint8)
    ro_mem = torch.arange(128, dtype=torch.uint8)
    seg = b.register(mem, token=41)
    ro = b.register(ro_mem, access=urma.READ, token=42)
    env = dict(urma=urma, a=a, b=b, ea=ea, peer=a.import_endpoint(eb.blob, token=3), mem=mem,
               rseg=a.import_segment(seg.blob, token=41), bad=a.import_segment(seg.blob, token=999),
               rro=a.import_segment(ro.blob, token=42), ro_mem=ro_mem)
    yield env
    a.close()
    b.close()


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(seq=st.lists(op, min_size=1, max_size=25))
def test_random_sequences_match_the_model(world, seq):
    urma, ea, peer, mem, rseg = world["urma"], world["ea"], world["peer"], world["mem"], world["rseg"]
    model = bytearray(mem.numpy().tobytes())
    for kind, x, y, z in seq:
        if kind == "write":
            n = min(y, SEG_BYTES - x)
            src = torch.full((n,), z, dtype=torch.uint8)
            ea.write(peer, rseg, rseg.va + x, src.data_ptr(), n)
            c = ea.wait(1)
            assert c[0].status == urma.CR_SUCCESS
            model[x:x + n] = bytes([z]) * n
        elif kind == "read":
            n = min(y, SEG_BYTES - x)
            dst = torch.zeros(n, dtype=torch.uint8)
            ea.read(peer, rseg, rseg.va + x, dst.data_ptr(), n)
            ea.wait(1)
            assert dst.numpy().tobytes() == bytes(model[x:x + n])
        elif kind == "fadd":
            old = ea.fetch_add(peer, rseg, rseg.va + 8 * x, y)
            want = int.from_bytes(model[8 * x:8 * x + 8], "little")
            assert old == want
            model[8 * x:8 * x + 8] = ((want + y) & ((1 << 64) - 1)).to_bytes(8, "little")
        elif kind == "cas":
            cur = int.from_bytes(model[8 * x:8 * x + 8], "little")
            old = ea.compare_swap(peer, rseg, rseg.va + 8 * x, y, z)
            assert old == cur
            if cur == y:
                model[8 * x:8 * x + 8] = z.to_bytes(8, "little")
        elif kind == "oob_write":
            src = torch.zeros(y, dtype=torch.uint8)
            ea.write(peer, rseg, rseg.va + x, src.data_ptr(), y)
            c = ea.wait(1, check=False)
            if x + y > SEG_BYTES:
                assert len(c) == 1 and c[0].status != urma.CR_SUCCESS
                with pytest.raises(urma.UrmaError):          # the jetty is in the ERROR state until recovered
                    ea.read(peer, rseg, rseg.va, src.data_ptr(), 8)
                ea.recover()
            else:
                assert c[0].status == urma.CR_SUCCESS
                model[x:x + y] = bytes(y)
        elif kind == "bad_token_write":
            src = torch.full((y,), 0xEE, dtype=torch.uint8)
            ea.write(peer, world["bad"], world["bad"].va + x, src.data_ptr(), y)
            c = ea.wait(1, check=False)
            assert len(c) == 1 and c[0].status == urma.CR_REM_ACCESS_ABORT
            ea.recover()
        elif kind == "ro_write":
            src = torch.full((y,), 0xDD, dtype=torch.uint8)
            ea.write(peer, world["rro"], world["rro"].va + x, src.data_ptr(), y)
            c = ea.wait(1, check=False)
            assert len(c) == 1 and c[0].status != urma.CR_SUCCESS
            ea.recover()
    assert mem.numpy().tobytes() == bytes(model)
    assert world["ro_mem"].tolist() == list(range(128))
    assert ea.poll(16) == []          # every completion was consumed; nothing spurious is queued
