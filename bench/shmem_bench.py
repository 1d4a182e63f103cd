#!/usr/bin/env python
"""Put bandwidth over the symmetric heap (torchrun, one rank per GPU; with one rank the destination is local memory).
Every rank copies rows of `row_bytes` into scattered rows of its right neighbour's heap with each access pattern of
`umdk_shmem_put_bench`; all ranks send at once, so the number is the per-direction link rate under full-duplex load. Device-timed, max over ranks."""
from __future__ import annotations

import argparse
import ctypes
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from bench.ep_bench import emit, setup, timed  # noqa: E402

MODES = {0: "stream of 16 B stores", 1: "warp per row, 16 B loads + stores",
         2: "warp per row, shared-memory stage + bulk store", 3: "warp per row, bulk load + bulk store"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mbytes", type=int, default=256)
    ap.add_argument("--row-bytes", type=int, nargs="*", default=[14336, 7168])
    ap.add_argument("--pieces", type=int, nargs="*", default=[2048, 4096, 7168])
    ap.add_argument("--grids", type=int, nargs="*", default=[148])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world = setup()
    from umdk_b200 import _native
    from umdk_b200.parallel.symm import SymmetricHeap
    lib = _native.cam()
    nbytes = a.mbytes << 20
    heap = SymmetricHeap(nbytes, None) if world > 1 else SymmetricHeap(nbytes)
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    peer = heap.peer_ptrs[(rank + 1) % world]
    lib.umdk_shmem_put_bench.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    for rb in a.row_bytes:
        rows = nbytes // rb
        for grid in a.grids:
            for mode in (0, 1, 2, 3):
                for piece in (a.pieces if mode >= 2 else [0]):
                    if mode >= 2 and piece > rb:
                        continue

                    def fn():
                        rc = lib.umdk_shmem_put_bench(peer, src.data_ptr(), rows, rb, piece, mode, grid,
                                                      status.data_ptr(), _native.stream_ptr())
                        assert rc == 0, rc
                    t = timed(fn, a.iters, a.warmup, world)
                    assert status.tolist()[0] == 0, status.tolist()
                    emit(rank, {"config": "shmem_put", "n_gpus": world, "row_bytes": rb, "grid": grid,
                                "pattern": MODES[mode], "piece": piece, "us": t * 1e6,
                                "GBps_per_direction": rows * rb / t / 1e9})
    heap.close()


if __name__ == "__main__":
    main()
