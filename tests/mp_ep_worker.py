"""Multi-process EP check, one rank per GPU (run under torchrun). Every rank regenerates all ranks' inputs from the
seed, runs the real kernels over NVLink peer memory, and compares its own outputs with the PyTorch oracle."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from umdk_b200.ops import reference as ref  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from umdk_b200.ops.ep import EpNormal
    from umdk_b200.ops.ep_ll import EpLowLatency, ExpertWeights
    from umdk_b200.parallel.symm import SymmetricHeap
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_ep_normal_gpu import _make_inputs
    from test_ep_ll_gpu import _inputs, _weights

    R = world
    # ---- normal mode ----
    T, H, E, K = 192, 2048, 8 * R, 4
    xs, idxs, ws = _make_inputs(R, T, H, E, K, seed=11, drop=True)
    heap = SymmetricHeap(EpNormal.heap_bytes(R, E, K, H, T))
    st = EpNormal(heap, E, K, H, T)
    x, idx, w = xs[rank].cuda(), idxs[rank].cuda(), ws[rank].cuda()
    want = ref.ref_dispatch_all(xs, idxs, ws, E, True)
    dist.barrier()   # the CPU oracle above takes each rank a different time
    for rnd in range(3):
        out = st.dispatch(x, idx, w, quant=True, sync_counts=True)
        n = out.num_recv
        assert n == want[rank].recv_x.shape[0], (n, want[rank].recv_x.shape)
        assert torch.equal(out.expand_idx[:n].cpu(), want[rank].expand_idx)
        assert torch.equal(out.recv_scales[:n].cpu(), want[rank].recv_scales)
        mism = (out.recv_x[:n].cpu().view(torch.uint8) != want[rank].recv_x.view(torch.uint8)).float().mean().item()
        assert mism < 5e-3, mism
        le = torch.repeat_interleave(torch.arange(E // R), want[rank].recv_tokens_per_expert)
        y = (ref.dequant_fp8_1x128(want[rank].recv_x, want[rank].recv_scales) *
             (le + rank * (E // R) + 1).float().unsqueeze(1)).to(torch.bfloat16)
        ybuf = torch.zeros(out.recv_x.shape[0], H, dtype=torch.bfloat16, device="cuda")
        ybuf[:n] = y.cuda()
        res = st.combine(ybuf, out)
        torch.cuda.synchronize()
        st.check("normal")
        ys = []
        for r in range(R):
            le_r = torch.repeat_interleave(torch.arange(E // R), want[r].recv_tokens_per_expert)
            ys.append((ref.dequant_fp8_1x128(want[r].recv_x, want[r].recv_scales) *
                       (le_r + r * (E // R) + 1).float().unsqueeze(1)).to(torch.bfloat16))
        want_c = ref.ref_combine_all(ys, want, idxs, ws, out_dtype=torch.float32)
        err = ref.mean_rel_err(res.float().cpu(), want_c[rank])
        assert err < 5e-3, err
    dist.barrier()
    heap.close()

    # ---- low-latency fused MoE ----
    T, H, F, E, K = 48, 1024, 512, 8 * R, 4
    w1q, w1s, w2q, w2s = _weights(E, H, F, seed=3)
    xs, idxs, ws = _inputs(R, T, H, E, K, seed=17)
    heap = SymmetricHeap(EpLowLatency.heap_bytes(R, E, K, H, T))
    ll = EpLowLatency(heap, E, K, H, F, T)
    el = E // R
    wt = ExpertWeights(*(t[rank * el:(rank + 1) * el].cuda().contiguous() for t in (w1q, w1s, w2q, w2s)))
    want = ref.ref_fused_moe(xs[rank], idxs[rank], ws[rank], w1q, w1s, w2q, w2s)
    x, idx, w = xs[rank].cuda(), idxs[rank].cuda(), ws[rank].cuda()
    dist.barrier()   # the CPU reference above takes each rank a different time
    for rnd in range(4):
        out, _, cnt = ll.moe(x, idx, w, wt)
        torch.cuda.synchronize()
        ll.check("ll")
        err = ref.mean_rel_err(out.float().cpu(), want)
        assert err < 0.012 and ref.max_row_rel_err(out.float().cpu(), want) < 0.05, err
    dist.barrier()
    heap.close()
    if rank == 0:
        print(f"MP_EP_OK world={world}")
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
