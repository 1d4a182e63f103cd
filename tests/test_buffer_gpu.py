"""GPU tests of the DeepEP-shaped Buffer front end on one rank: the default dispatch (host reads the counts), the
form that keeps every count on the device, and a buffer that is destroyed and built again between calls."""
import pytest
import torch

from umdk_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

T, H, E, K = 200, 1024, 16, 4


def _inputs(seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w, idx = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), K, dim=-1)
    idx[::9, 1] = -1
    return x, idx.to(torch.int64), (w / w.sum(-1, keepdim=True)).float()


def _check_dispatch(buf, x, idx, w, static):
    want = ref.ref_dispatch_all([x], [idx], [w], E, True)[0]
    n = want.recv_x.shape[0]
    (rx, rs), rows_le, rw, per_expert, handle, _ = buf.dispatch(
        x.cuda(), topk_idx=idx.cuda(), topk_weights=w.cuda(), num_experts=E, static_shapes=static)
    torch.cuda.synchronize()
    if static:
        assert isinstance(per_expert, torch.Tensor) and rx.shape[0] >= n
        assert per_expert.cpu().tolist() == want.recv_tokens_per_expert.tolist()
        assert (rows_le[n:] == -1).all() and (rw[n:] == 0).all()
    else:
        assert rx.shape[0] == n and per_expert == want.recv_tokens_per_expert.tolist()
    # fp8 rounding of x * (448 / amax): identical arithmetic, a rare 1-ulp tie difference is allowed
    mism = (rx[:n].view(torch.uint8).cpu() != want.recv_x.view(torch.uint8)).float().mean().item()
    assert mism < 5e-3, mism
    assert torch.equal(rs[:n].cpu(), want.recv_scales)
    assert torch.equal(rw[:n].cpu(), want.recv_weights)
    le = torch.repeat_interleave(torch.arange(E), want.recv_tokens_per_expert)
    assert torch.equal(rows_le[:n].cpu(), le)
    # combine what was received (an identity expert): out[t] = sum_k w[t,k] * dequant(x[t])
    y = torch.zeros(rx.shape[0], H, dtype=torch.bfloat16, device="cuda")
    y[:n] = ref.dequant_fp8_1x128(want.recv_x, want.recv_scales).to(torch.bfloat16).cuda()
    out, _, _ = buf.combine(y, handle)
    torch.cuda.synchronize()
    want_out = ref.ref_combine_all([y[:n].cpu()], [want], [idx], [w])[0]
    assert ref.mean_rel_err(out.float().cpu(), want_out.float()) < 5e-3


def test_buffer_dispatch_with_and_without_host_sync():
    from umdk_b200.buffer import Buffer
    buf = Buffer(None, max_tokens_per_rank=T)
    try:
        x, idx, w = _inputs(1)
        _check_dispatch(buf, x, idx, w, static=False)
        _check_dispatch(buf, x, idx, w, static=True)
        buf.static_shapes = True   # the attribute selects the same form
        res = buf.dispatch(x.cuda(), topk_idx=idx.cuda(), topk_weights=w.cuda(), num_experts=E)
        assert isinstance(res[3], torch.Tensor)
    finally:
        buf.destroy()


def test_buffer_destroy_recreate_dispatch():
    """A rank that restarts builds its buffer again: the new one must work from a clean protocol state (epochs,
    flags, counters) no matter what the old one left behind."""
    from umdk_b200.buffer import Buffer
    for life in range(3):
        buf = Buffer(None, max_tokens_per_rank=T)
        x, idx, w = _inputs(10 + life)
        for _ in range(life + 1):          # a different number of calls per life: epochs differ at destroy time
            _check_dispatch(buf, x, idx, w, static=False)
        buf.destroy()
        assert not buf._normal and not buf._ll
