"""Device-side symmetric-memory API (csrc/cam/shmem_device.cuh): put / get / quiet / signal / atomics against peer
heaps, on several processing elements that share one GPU (send phases of all PEs run before any wait phase), and a
wait that nothing satisfies, which must return its status within the cycle budget instead of hanging."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, heaps, r, phase, tag, limit, result):
    R = len(heaps)
    arr = (ctypes.c_void_p * R)(*heaps[r].peer_ptrs)
    rc = lib.umdk_shmem_selftest(arr, R, r, ctypes.c_uint64(heaps[r].nbytes), phase, ctypes.c_uint64(tag),
                                 ctypes.c_longlong(limit), ctypes.c_void_p(result.data_ptr()), None)
    assert rc == 0


@pytest.mark.parametrize("R", [1, 2, 4, 8])
def test_shmem_ops_virtual_pes(R):
    from umdk_b200 import _native
    from umdk_b200.parallel.symm import SymmetricHeap
    lib = _native.cam()
    heaps = SymmetricHeap.virtual(1 << 16, R)
    try:
        from umdk_b200.utils.rawtensor import from_ptr
        dev = torch.device("cuda", torch.cuda.current_device())
        for h in heaps:
            from_ptr(h.local_ptr, (h.nbytes,), torch.uint8, dev).zero_()
        # word 3 of the 32-bit atomics starts as all-ones so that the AND of every PE clears one bit each
        a32 = from_ptr(heaps[0].local_ptr + 17408 + 512, (4,), torch.int32, dev)
        a32[3] = -1
        res = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(R)]
        for r in range(R):
            _run(lib, heaps, r, 1, 7, 1 << 30, res[r])
        for r in range(R):
            _run(lib, heaps, r, 2, 7, 1 << 30, res[r])
        torch.cuda.synchronize()
        out = [t.cpu().tolist() for t in res]
        full = (1 << R) - 1
        for r in range(R):
            assert out[r][0] == 0, out[r]
            assert out[r][1] == R * (R + 1) // 2            # add
            assert out[r][2] == full                        # or
            assert out[r][3] == full                        # xor of distinct bits
            assert out[r][6] == R                           # inc
            assert (out[r][7] & 0xFFFF) == (0xFFFF & ~full)  # and
        assert sorted(o[5] for o in out) == list(range(R))  # fetch_inc hands out distinct tickets
        assert sum(1 for o in out if o[4] == 0) == 1        # exactly one compare-and-swap saw the initial value
    finally:
        for h in heaps:
            h.close()


def test_shmem_wait_times_out_with_status():
    from umdk_b200 import _native
    from umdk_b200.parallel.symm import SymmetricHeap
    lib = _native.cam()
    heaps = SymmetricHeap.virtual(1 << 16, 1)
    try:
        from umdk_b200.utils.rawtensor import from_ptr
        from_ptr(heaps[0].local_ptr, (heaps[0].nbytes,), torch.uint8,
                 torch.device("cuda", torch.cuda.current_device())).zero_()
        res = torch.zeros(16, dtype=torch.int32, device="cuda")
        _run(lib, heaps, 0, 3, 1, 2_000_000, res)   # about a millisecond of budget
        torch.cuda.synchronize()
        out = res.cpu().tolist()
        assert out[8] == 0 and out[9] >= 1900
        # the context is still usable
        assert int(torch.arange(10, device="cuda").sum().item()) == 45
    finally:
        heaps[0].close()


@pytest.mark.parametrize("mode,piece", [(0, 0), (1, 0), (2, 2048), (2, 7168), (3, 4096), (3, 14336)])
def test_put_patterns_copy_every_row(mode, piece):
    """Each access pattern of the put-bandwidth probe moves every row to its scattered destination row."""
    import ctypes
    from umdk_b200 import _native
    lib = _native.cam()
    rows, rb = 1000, 14336
    src = torch.randint(0, 255, (rows, rb), dtype=torch.uint8, device="cuda")
    dst = torch.zeros_like(src)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    lib.umdk_shmem_put_bench.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    rc = lib.umdk_shmem_put_bench(dst.data_ptr(), src.data_ptr(), rows, rb, piece, mode, 16, status.data_ptr(),
                                  _native.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    if mode == 0:
        assert torch.equal(dst, src)
    else:
        perm = (torch.arange(rows) * 9973 + 17) % rows
        assert torch.equal(dst[perm.cuda()], src)
