"""GPU tests of the normal-mode EP kernels against the PyTorch oracle. Several ranks are emulated on one GPU by
running the send half of every rank before any receive half (kernels that wait on each other never run as
separate launches)."""
import pytest
import torch

from umdk_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _make_inputs(R, T, H, E, K, seed=0, drop=False):
    g = torch.Generator().manual_seed(seed)
    xs, idxs, ws = [], [], []
    for r in range(R):
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, generator=g)
        p = torch.softmax(logits, dim=-1)
        w, idx = torch.topk(p, K, dim=-1)
        w = (w / w.sum(dim=-1, keepdim=True)).float()
        if drop:
            idx[::7, 0] = -1
        xs.append(x)
        idxs.append(idx.to(torch.int64))
        ws.append(w)
    return xs, idxs, ws


def _virtual_states(R, E, K, H, cap):
    from umdk_b200.ops.ep import EpNormal
    from umdk_b200.parallel.symm import SymmetricHeap
    nbytes = EpNormal.heap_bytes(R, E, K, H, cap)
    heaps = SymmetricHeap.virtual(nbytes, R)
    return heaps, [EpNormal(h, E, K, H, cap) for h in heaps]


@pytest.mark.parametrize("T,K,E,R", [(1, 1, 8, 1), (37, 2, 16, 2), (300, 8, 64, 8), (4096, 8, 256, 8)])
def test_layout_matches_reference(T, K, E, R):
    from umdk_b200.ops.ep import layout
    _, idxs, _ = _make_inputs(1, T, 128, E, K, seed=T, drop=(T > 10))
    got = layout(idxs[0].cuda(), E, R)
    want = ref.ref_layout(idxs[0], E, R)
    torch.cuda.synchronize()
    assert torch.equal(got.num_tokens_per_expert.cpu(), want.num_tokens_per_expert)
    assert torch.equal(got.num_tokens_per_rank.cpu(), want.num_tokens_per_rank)
    assert torch.equal(got.is_token_in_rank.cpu(), want.is_token_in_rank)
    assert torch.equal(got.send_token_idx.cpu(), want.send_token_idx)
    assert torch.equal(got.rank_slot.cpu(), want.rank_slot)
    # the same call into the tensors of the earlier result (no allocations on the call path)
    idx2 = torch.roll(idxs[0], 3, 0)
    again = layout(idx2.cuda(), E, R, out=got)
    want2 = ref.ref_layout(idx2, E, R)
    torch.cuda.synchronize()
    assert again is got and torch.equal(got.send_token_idx.cpu(), want2.send_token_idx)
    assert torch.equal(got.is_token_in_rank.cpu(), want2.is_token_in_rank)


@pytest.mark.parametrize("R,T,H,E,K,quant", [
    (1, 64, 1024, 8, 2, True),
    (2, 128, 1024, 16, 2, True),
    (2, 128, 1024, 16, 2, False),
    (4, 257, 2048, 32, 4, True),
    (8, 96, 7168, 256, 8, True),
])
def test_dispatch_combine_virtual_ranks(R, T, H, E, K, quant):
    xs, idxs, ws = _make_inputs(R, T, H, E, K, seed=R * 1000 + T, drop=True)
    heaps, states = _virtual_states(R, E, K, H, cap=T)
    try:
        dx = [x.cuda() for x in xs]
        di = [i.cuda() for i in idxs]
        dw = [w.cuda() for w in ws]
        # two rounds: the second exercises the epoch / ping-pong logic
        for rnd in range(2):
            outs = [states[r].dispatch(dx[r], di[r], dw[r], quant=quant, phase_mask=1) for r in range(R)]
            outs = [states[r].dispatch(dx[r], di[r], dw[r], quant=quant, phase_mask=2, out=outs[r]) for r in range(R)]
            torch.cuda.synchronize()
            for s in states:
                s.check("dispatch")
            want = ref.ref_dispatch_all(xs, idxs, ws, E, quant)
            ys = []
            for r in range(R):
                n = int(outs[r].counts[0].item())
                assert n == want[r].recv_x.shape[0]
                assert torch.equal(outs[r].recv_count.cpu(), want[r].recv_count)
                assert torch.equal(outs[r].recv_tokens_per_expert.cpu(), want[r].recv_tokens_per_expert)
                assert torch.equal(outs[r].expand_idx[:n].cpu(), want[r].expand_idx)
                if quant:
                    assert torch.equal(outs[r].recv_scales[:n].cpu(), want[r].recv_scales)
                    got = outs[r].recv_x[:n].cpu().view(torch.uint8)
                    exp = want[r].recv_x.view(torch.uint8)
                    # fp8 rounding of x * (448 / amax): identical arithmetic, allow a rare 1-ulp tie difference
                    mism = (got != exp).float().mean().item()
                    assert mism < 5e-3, mism
                else:
                    assert torch.equal(outs[r].recv_x[:n].cpu(), want[r].recv_x)
                # "expert" = identity * (global expert id + 1)
                le = torch.repeat_interleave(torch.arange(E // R), want[r].recv_tokens_per_expert)
                scale = (le + r * (E // R) + 1).float().unsqueeze(1)
                if quant:
                    xin = ref.dequant_fp8_1x128(want[r].recv_x, want[r].recv_scales)
                else:
                    xin = want[r].recv_x.float()
                y = (xin * scale).to(torch.bfloat16)
                ybuf = torch.zeros(outs[r].recv_x.shape[0], H, dtype=torch.bfloat16, device="cuda")
                ybuf[:n] = y.cuda()
                ys.append((y, ybuf))
            res = [None] * R
            for r in range(R):
                res[r] = states[r].combine(ys[r][1], outs[r], phase_mask=1)
            for r in range(R):
                res[r] = states[r].combine(ys[r][1], outs[r], phase_mask=2, out=res[r])
            torch.cuda.synchronize()
            for s in states:
                s.check("combine")
            want_c = ref.ref_combine_all([y for y, _ in ys], want, idxs, ws, out_dtype=torch.float32)
            for r in range(R):
                err = ref.mean_rel_err(res[r].float().cpu(), want_c[r])
                assert err < 5e-3, (r, err)
            # row-per-(token,k) combine (reference contract)
            res2 = [None] * R
            for r in range(R):
                n = want[r].recv_x.shape[0]
                res2[r] = states[r].combine_rows(ys[r][1][:n].contiguous(), outs[r].expand_idx[:n].contiguous(),
                                                 di[r], dw[r], phase_mask=1)
            for r in range(R):
                n = want[r].recv_x.shape[0]
                res2[r] = states[r].combine_rows(ys[r][1][:n].contiguous(), outs[r].expand_idx[:n].contiguous(),
                                                 di[r], dw[r], phase_mask=2, out=res2[r])
            torch.cuda.synchronize()
            for s in states:
                s.check("combine_rows")
            for r in range(R):
                err = ref.mean_rel_err(res2[r].float().cpu(), want_c[r])
                assert err < 5e-3, (r, err)
    finally:
        for h in heaps:
            h.close()


def test_diagnose_mode_records_wait_times():
    """With diagnose on, dispatch and combine fill one wait time per source rank (non-negative, small on one GPU)."""
    from umdk_b200.ops.ep import EpNormal
    from umdk_b200.parallel.symm import SymmetricHeap
    R, T, H, E, K = 1, 64, 512, 8, 2
    heap = SymmetricHeap(EpNormal.heap_bytes(R, E, K, H, T))
    try:
        st = EpNormal(heap, E, K, H, T)
        st.diagnose = True
        st.diag_dispatch.fill_(-1)
        st.diag_combine.fill_(-1)
        g = torch.Generator().manual_seed(0)
        x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
        idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int64).cuda()
        w = torch.full((T, K), 0.5).cuda()
        d = st.dispatch(x, idx, w, quant=False, sync_counts=True)
        y = d.recv_x[:d.num_recv].view(torch.bfloat16).reshape(d.num_recv, H).contiguous()
        out = st.combine(y, d)
        torch.cuda.synchronize()
        wd, wc = st.wait_times_us()
        assert (wd >= 0).all() and (wc >= 0).all() and float(wd.max()) < 1e6
        assert ref.mean_rel_err(out.float().cpu(), x.float().cpu()) < 1e-2
    finally:
        heap.close()


@pytest.mark.parametrize("R,T,E,K", [(1, 64, 8, 2), (2, 128, 16, 2), (8, 300, 256, 8)])
def test_notify_matches_dispatch_counts(R, T, E, K):
    """The standalone count exchange gives the numbers dispatch derives internally, and can be interleaved with it."""
    H = 1024
    xs, idxs, ws = _make_inputs(R, T, H, E, K, seed=R * 31 + T, drop=True)
    heaps, states = _virtual_states(R, E, K, H, cap=T)
    try:
        di = [i.cuda() for i in idxs]
        el = E // R
        for rnd in range(3):
            lays = [states[r].layout(di[r]) for r in range(R)]
            outs = [states[r].notify(lays[r], phase_mask=1) for r in range(R)]
            outs = [states[r].notify(lays[r], phase_mask=2, out=outs[r]) for r in range(R)]
            if rnd == 1:  # a dispatch in between must not disturb the operator's own epoch
                d = [states[r].dispatch(xs[r].cuda(), di[r], ws[r].cuda(), phase_mask=1) for r in range(R)]
                d = [states[r].dispatch(xs[r].cuda(), di[r], ws[r].cuda(), phase_mask=2, out=d[r]) for r in range(R)]
            torch.cuda.synchronize()
            want_lay = [ref.ref_layout(i, E, R) for i in idxs]
            for r in range(R):
                states[r].check("notify")
                cnt = torch.stack([want_lay[s].num_tokens_per_expert[r * el:(r + 1) * el] for s in range(R)])  # [src, le]
                flat = cnt.t().reshape(-1).to(torch.int64)
                incl = torch.cumsum(flat, 0)
                assert torch.equal(outs[r].recv_count.cpu().long(), incl)
                assert torch.equal(outs[r].recv_offset.cpu().long(), incl - flat)
                assert torch.equal(outs[r].recv_tokens_per_expert.cpu(), cnt.sum(0).to(torch.int64))
                arr = [int(want_lay[s].num_tokens_per_rank[r]) for s in range(R)]
                assert outs[r].totals.tolist()[:3] == [int(flat.sum()), sum(arr), max(arr)]
                if rnd == 1:
                    assert torch.equal(d[r].recv_count.cpu(), outs[r].recv_count.cpu())
            idxs = [torch.roll(i, 1, 0) for i in idxs]
            di = [i.cuda() for i in idxs]
    finally:
        for h in heaps:
            h.close()
