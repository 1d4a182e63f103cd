"""The allocation-free layout entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory when they need a routing layout: an inference server
that gave all free memory to its KV-cache pool at start-up, or an op that runs inside another runtime's enqueue hook
where allocation is not permitted. For them ``umdk_ep_layout_noalloc`` keeps its scratch in a fixed array inside
the library. This test loads the shared library with plain ctypes (no package wrapper in between), calls the symbol
twice in a row on different inputs - the second call sees whatever the first one left in the shared array - and
requires exactly the same integers as the ordinary entry point, which gets freshly allocated scratch.
This file sorts last on purpose so that a run which stops at the first failure has already run everything else.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "umdk_b200", "_lib",
                   "libumdk_cam.so")


def _topk(T, K, E, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.topk(torch.rand(T, E, generator=g), K, dim=-1).indices.to(torch.int64)
    idx[::9, K - 1] = -1
    return idx


def _call_noalloc(lib, idx, E, R):
    T, K = idx.shape
    dev = idx.device
    out = dict(npe=torch.empty(E, dtype=torch.int32, device=dev), npr=torch.empty(R, dtype=torch.int32, device=dev),
               inr=torch.empty(T, R, dtype=torch.uint8, device=dev), sidx=torch.empty(T, K, dtype=torch.int32, device=dev),
               rslot=torch.empty(T, R, dtype=torch.int32, device=dev))
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.umdk_ep_layout_noalloc(p(idx), T, K, E, R, p(out["npe"]), p(out["npr"]), p(out["inr"]), p(out["sidx"]),
                                    p(out["rslot"]), p(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out, status


def _load():
    from umdk_b200 import _native
    _native.cam()          # builds the library on a fresh checkout; the symbol itself is called through plain ctypes
    lib = ctypes.CDLL(LIB)
    lib.umdk_ep_layout_noalloc.restype = ctypes.c_int
    return lib


def test_noalloc_layout_matches_regular_entry_point_twice():
    from umdk_b200.ops.ep import layout
    lib = _load()
    for call, (T, K, E, R) in enumerate([(4096, 8, 256, 8), (777, 4, 64, 4)]):
        idx = _topk(T, K, E, seed=call).cuda()
        rc, got, status = _call_noalloc(lib, idx, E, R)
        assert rc == 0
        want = layout(idx, E, R)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        assert torch.equal(got["npe"], want.num_tokens_per_expert)
        assert torch.equal(got["npr"], want.num_tokens_per_rank)
        assert torch.equal(got["inr"].view(torch.bool), want.is_token_in_rank)
        assert torch.equal(got["sidx"], want.send_token_idx)
        assert torch.equal(got["rslot"], want.rank_slot)


def test_noalloc_layout_takes_no_device_memory_after_its_first_call():
    """Free device memory as the driver reports it is the same before and after the second and third call: the
    claim a caller whose pool owns every free byte relies on. (The first call may load the module.)"""
    lib = _load()
    idx = _topk(2048, 8, 128, seed=11).cuda()
    rc, _, _ = _call_noalloc(lib, idx, 128, 8)
    assert rc == 0
    torch.cuda.synchronize()
    dev = idx.device
    bufs = dict(npe=torch.empty(128, dtype=torch.int32, device=dev), npr=torch.empty(8, dtype=torch.int32, device=dev),
                inr=torch.empty(2048, 8, dtype=torch.uint8, device=dev),
                sidx=torch.empty(2048, 8, dtype=torch.int32, device=dev),
                rslot=torch.empty(2048, 8, dtype=torch.int32, device=dev))
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        rc = lib.umdk_ep_layout_noalloc(p(idx), 2048, 8, 128, 8, p(bufs["npe"]), p(bufs["npr"]), p(bufs["inr"]),
                                        p(bufs["sidx"]), p(bufs["rslot"]), p(status), stream)
        assert rc == 0
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert free1 == free0
    assert status.tolist()[0] == 0 and int(bufs["npe"].sum()) == int((idx >= 0).sum())


def test_noalloc_layout_rejects_sizes_beyond_its_scratch():
    lib = _load()
    idx = _topk(64, 2, 16, seed=3).cuda()
    null = ctypes.c_void_p(0)
    # token count above the limit: refused before anything is launched (outputs are never touched)
    rc = lib.umdk_ep_layout_noalloc(ctypes.c_void_p(idx.data_ptr()), 8193, 2, 16, 2, null, null, null, null, null,
                                    null, null)
    assert rc == -2
    rc = lib.umdk_ep_layout_noalloc(ctypes.c_void_p(idx.data_ptr()), 64, 2, 1024, 32, null, null, null, null, null,
                                    null, null)
    assert rc == -2
