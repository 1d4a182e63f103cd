"""Multi-process check of the tensor-parallel kernels, the all-reduce variants (peer loads and NVLS multimem) and the
URMA cuda_ipc provider across real GPUs (run under torchrun, one rank per GPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from umdk_b200.ops.tp import AllReduce, TpComm
    from umdk_b200.parallel.symm import SymmetricHeap
    R = world
    Ts, K, N = 256, 1024, 512
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(Ts, K, generator=g).to(torch.bfloat16) for _ in range(R)]
    ws = [(torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16) for _ in range(R)]
    ys = [torch.randn(R * Ts, K, generator=g).to(torch.bfloat16) for _ in range(R)]
    wd = [(torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16) for _ in range(R)]
    heap = SymmetricHeap(TpComm.heap_bytes(R, Ts, K, N))
    tp = TpComm(heap, Ts, K, N, n_copy=8)
    for rnd in range(4):
        out = tp.ag_gemm((xs[rank] + rnd).cuda(), ws[rank].cuda())
        o2 = tp.gemm_rs(ys[rank].cuda() * (rnd + 1), wd[rank].cuda())
        torch.cuda.synchronize()
        tp.check()
        xall = torch.cat([x + rnd for x in xs]).float()
        assert rel(out.cpu(), xall @ ws[rank].float().t()) < 5e-3
        full = sum((ys[s].float() * (rnd + 1)) @ wd[s].float().t() for s in range(R))
        assert rel(o2.cpu(), full[rank * Ts:(rank + 1) * Ts]) < 1e-2
    dist.barrier()
    heap.close()
    # all-reduce: peer-load algorithms on the IPC heap, NVLS on the multicast heap
    n = 1 << 20
    vals = [torch.randn(n, generator=g).to(torch.bfloat16) for _ in range(R)]
    want = sum(v.float() for v in vals)
    heap = SymmetricHeap(AllReduce.heap_bytes(n * 4, R))
    ar = AllReduce(heap, n * 4)
    for algo in ("one_shot", "two_shot", "push", "one_shot", "push", "push", "two_shot"):
        out = ar(vals[rank].cuda(), algo=algo)
        torch.cuda.synchronize()
        ar.check()
        assert rel(out.cpu(), want) < 1e-2, algo
    small = ar(vals[rank][:8 * R * 16].cuda().contiguous(), algo="one_shot")
    torch.cuda.synchronize()
    assert rel(small.cpu(), want[:8 * R * 16]) < 1e-2
    dist.barrier()
    heap.close()
    nvls = "skipped"
    if os.environ.get("UMDK_TEST_NVLS", "1") == "1":
        try:
            mheap = SymmetricHeap.multicast(AllReduce.heap_bytes(n * 2, R))
        except Exception as e:
            mheap = None
            nvls = f"unavailable ({type(e).__name__})"
        if mheap is not None:
            ar = AllReduce(mheap, n * 2)
            for _ in range(3):
                out = ar(vals[rank].cuda(), algo="nvls")
                torch.cuda.synchronize()
                ar.check()
                assert rel(out.cpu(), want) < 1e-2
            buf = ar.buffer(n, ar.next_parity)
            buf.copy_(vals[rank].cuda())
            ar(None, algo="nvls", in_place=True, n=n)
            torch.cuda.synchronize()
            ar.check()
            assert rel(buf.cpu(), want) < 1e-2
            nvls = "ok"
            dist.barrier()
    # URMA over GPU memory across processes (CUDA IPC handles through the provider's directory)
    from umdk_b200 import urma
    ctx = urma.Context(f"cuda{torch.cuda.current_device()}")
    ep = ctx.endpoint(depth=32)
    mem = torch.zeros(4096, dtype=torch.float32, device="cuda")
    seg = ctx.register(mem, token=40 + rank)
    blobs = [None] * R
    dist.all_gather_object(blobs, (ep.blob, seg.blob))
    peer = (rank + 1) % R
    # different GPUs are different URMA devices; the target handle only names the destination
    tj = ctx.import_endpoint(blobs[peer][0])
    rseg = ctx.import_segment(blobs[peer][1], token=40 + peer)
    src = torch.full((1024,), float(rank + 1), device="cuda")
    ep.write(tj, rseg, rseg.va, src.data_ptr(), 4096)
    ep.wait(1)
    dist.barrier()
    torch.cuda.synchronize()
    assert torch.equal(mem[:1024].cpu(), torch.full((1024,), float((rank - 1) % R + 1)))
    dist.barrier()
    ctx.close()
    if rank == 0:
        print(f"MP_TP_OK world={world} nvls={nvls}")
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException as e:   # the launcher only keeps the tail of the output: say what failed in one line
        import traceback
        tb = traceback.extract_tb(e.__traceback__)[-1]
        print(f"MP_WORKER_ERROR rank={os.environ.get('RANK')} {type(e).__name__}: {str(e)[:300]} "
              f"at {os.path.basename(tb.filename)}:{tb.lineno}", flush=True)
        raise
