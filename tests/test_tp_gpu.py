"""Tensor-parallel fused kernels against fp32 PyTorch references. Several ranks are emulated on one GPU by running
each communication phase for every rank in turn (publish / push first, wait / reduce second)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


# shapes with Ts and N multiples of 256 run on CTA pairs unless single_cta is set; the others always on one CTA per tile
@pytest.mark.parametrize("single_cta", [False, True])
@pytest.mark.parametrize("R,Ts,K,N", [(1, 128, 256, 256), (2, 128, 512, 512), (4, 256, 1024, 768), (2, 512, 512, 512)])
def test_allgather_gemm(R, Ts, K, N, single_cta):
    from umdk_b200.ops.tp import TpComm
    from umdk_b200.parallel.symm import SymmetricHeap
    g = torch.Generator().manual_seed(R)
    xs = [torch.randn(Ts, K, generator=g).to(torch.bfloat16).cuda() for _ in range(R)]
    ws = [(torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda() for _ in range(R)]
    heaps = SymmetricHeap.virtual(TpComm.heap_bytes(R, Ts, K, 256), R)
    try:
        comms = [TpComm(h, Ts, K, 256, n_copy=4, single_cta=single_cta) for h in heaps]
        for rnd in range(3):
            for r in range(R):
                comms[r].ag_gemm(xs[r], ws[r], phase_mask=4)
            outs = [comms[r].ag_gemm(xs[r], ws[r]) for r in range(R)]
            torch.cuda.synchronize()
            xall = torch.cat(xs).float()
            for r in range(R):
                comms[r].check()
                assert _rel(outs[r], xall @ ws[r].float().t()) < 5e-3
            xs = [x + 1 for x in xs]  # new data every round: stale shards would be noticed
    finally:
        for h in heaps:
            h.close()


@pytest.mark.parametrize("single_cta", [False, True])
@pytest.mark.parametrize("R,Ts,Kr,N", [(1, 128, 128, 256), (2, 128, 256, 512), (4, 128, 512, 256), (2, 256, 256, 512),
                                       (4, 512, 320, 256)])
def test_gemm_reduce_scatter(R, Ts, Kr, N, single_cta):
    from umdk_b200.ops.tp import TpComm
    from umdk_b200.parallel.symm import SymmetricHeap
    g = torch.Generator().manual_seed(10 + R)
    ys = [torch.randn(R * Ts, Kr, generator=g).to(torch.bfloat16).cuda() for _ in range(R)]
    ws = [(torch.randn(N, Kr, generator=g) * 0.05).to(torch.bfloat16).cuda() for _ in range(R)]
    heaps = SymmetricHeap.virtual(TpComm.heap_bytes(R, Ts, 256, N), R)
    try:
        comms = [TpComm(h, Ts, 256, N, single_cta=single_cta) for h in heaps]
        for rnd in range(3):
            outs = [comms[r].gemm_rs(ys[r], ws[r], phase_mask=1) for r in range(R)]
            for r in range(R):
                comms[r].gemm_rs(ys[r], ws[r], out=outs[r], phase_mask=2)
            torch.cuda.synchronize()
            full = sum(ys[s].float() @ ws[s].float().t() for s in range(R))
            for r in range(R):
                comms[r].check()
                assert _rel(outs[r], full[r * Ts:(r + 1) * Ts]) < 1e-2
            ys = [y * 0.5 + 0.25 for y in ys]
    finally:
        for h in heaps:
            h.close()


@pytest.mark.parametrize("R,n", [(1, 4096), (2, 1 << 16), (4, 1 << 18), (8, 64 * 1024)])
def test_one_shot_allreduce_virtual_ranks(R, n):
    from umdk_b200.ops.tp import AllReduce
    from umdk_b200.parallel.symm import SymmetricHeap
    g = torch.Generator().manual_seed(n)
    heaps = SymmetricHeap.virtual(AllReduce.heap_bytes(n * 2, R), R)
    try:
        ars = [AllReduce(h, n * 2) for h in heaps]
        for rnd in range(4):
            xs = [torch.randn(n, generator=g).to(torch.bfloat16).cuda() for _ in range(R)]
            outs = [ars[r](xs[r], algo="one_shot", phase_mask=1) for r in range(R)]
            for r in range(R):
                ars[r](xs[r], out=outs[r], algo="one_shot", phase_mask=2)
            torch.cuda.synchronize()
            want = sum(x.float() for x in xs)
            for r in range(R):
                ars[r].check()
                assert _rel(outs[r], want) < 1e-2
    finally:
        for h in heaps:
            h.close()


@pytest.mark.parametrize("R,n", [(1, 4096), (2, 1 << 16), (4, 1 << 18), (8, 64 * 1024)])
def test_push_allreduce_virtual_ranks(R, n):
    """Store-only two-shot: contributions pushed, slices reduced and pushed back, then copied out (three phases)."""
    from umdk_b200.ops.tp import AllReduce
    from umdk_b200.parallel.symm import SymmetricHeap
    g = torch.Generator().manual_seed(n + 1)
    heaps = SymmetricHeap.virtual(AllReduce.heap_bytes(n * 4, R), R)
    try:
        ars = [AllReduce(h, n * 4) for h in heaps]
        for rnd in range(4):
            xs = [torch.randn(n, generator=g).to(torch.bfloat16).cuda() for _ in range(R)]
            outs = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
            for phase in (1, 2, 4):
                for r in range(R):
                    ars[r](xs[r], out=outs[r], algo="push", phase_mask=phase)
            torch.cuda.synchronize()
            want = sum(x.float() for x in xs)
            for r in range(R):
                ars[r].check()
                assert _rel(outs[r], want) < 1e-2, (rnd, r)
    finally:
        for h in heaps:
            h.close()


@pytest.mark.parametrize("R,n", [(2, 4096), (4, 1 << 16), (8, 1 << 17)])
def test_one_shot_push_allreduce_virtual_ranks(R, n):
    from umdk_b200.ops.tp import AllReduce
    from umdk_b200.parallel.symm import SymmetricHeap
    g = torch.Generator().manual_seed(n + 2)
    heaps = SymmetricHeap.virtual(AllReduce.heap_bytes(n * 2 * R, R), R)
    try:
        ars = [AllReduce(h, n * 2 * R) for h in heaps]
        for rnd in range(4):
            xs = [torch.randn(n, generator=g).to(torch.bfloat16).cuda() for _ in range(R)]
            outs = [ars[r](xs[r], algo="one_shot_push", phase_mask=1) for r in range(R)]
            for r in range(R):
                ars[r](xs[r], out=outs[r], algo="one_shot_push", phase_mask=2)
            torch.cuda.synchronize()
            want = sum(x.float() for x in xs)
            for r in range(R):
                ars[r].check()
                assert _rel(outs[r], want) < 1e-2, (rnd, r)
    finally:
        for h in heaps:
            h.close()


def test_two_shot_allreduce_single_rank():
    from umdk_b200.ops.tp import AllReduce
    from umdk_b200.parallel.symm import SymmetricHeap
    n = 1 << 20
    heap = SymmetricHeap(AllReduce.heap_bytes(n * 2, 1))
    try:
        ar = AllReduce(heap, n * 2)
        x = torch.randn(n).to(torch.bfloat16).cuda()
        for _ in range(3):
            out = ar(x, algo="two_shot")
        torch.cuda.synchronize()
        ar.check()
        assert torch.equal(out, x)
    finally:
        heap.close()
