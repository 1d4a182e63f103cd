"""The operator library registered from C++ (csrc/torch_ext): schemas, Meta shape functions and the Autograd key; and
the two pieces of `fused_deep_moe` argument handling that run on the host (per-expert weight lists, smooth scales)."""
import pytest
import torch

import umdk_b200
from umdk_b200.ops import reference as ref

ops = umdk_b200.load_torch_ops()
lib = torch.ops.umdk_cam_op_lib


def _moe_args(T=64, H=1024, F=256, E=8, K=4, R=2, device="cpu", as_list=False):
    el = E // R
    w1 = torch.empty(el, 2 * F, H, dtype=torch.uint8, device=device).view(torch.float8_e4m3fn)
    s1 = torch.empty(el, 2 * F // 128, H // 128, device=device)
    w2 = torch.empty(el, H, F, dtype=torch.uint8, device=device).view(torch.float8_e4m3fn)
    s2 = torch.empty(el, H // 128, F // 128, device=device)
    lists = [list(t.unbind(0)) if as_list else [t] for t in (w1, s1, w2, s2)]
    x = torch.empty(T, H, dtype=torch.bfloat16, device=device)
    ids = torch.zeros(T, K, dtype=torch.int64, device=device)
    scales = torch.empty(T, K, device=device)
    return (x, ids, *lists, scales, None, None, None, None, None, None, None, "ep", R, 0, E, 0, T * R)


@pytest.mark.skipif(not ops.CPP_LIBRARY_LOADED, reason="C++ operator library not built")
def test_meta_shape_functions_serve_fake_tensor_tracing():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        out, share, cnt = lib.fused_deep_moe(*_moe_args(device="cuda", as_list=True))
        assert out.shape == (64, 1024) and share.shape == (64, 1024) and out.dtype == torch.bfloat16
        assert cnt.shape == (4,) and cnt.dtype == torch.int64 and out.device.type == "cuda"
        ids = torch.empty(100, 8, dtype=torch.int64, device="cuda")
        npe, sidx = lib.get_dispatch_layout(ids, 64, 8)
        assert npe.shape == (64,) and sidx.shape == (100, 8) and npe.dtype == torch.int32
        x = torch.empty(100, 2048, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(100, 8, device="cuda")
        rx, rs, ex, rc, rpe = lib.moe_dispatch_prefill(x, ids, w, npe, sidx, "ep", 0, 8, True)
        n = 8 * 100 * 8
        assert rx.shape == (n, 2048) and rx.dtype == torch.float8_e4m3fn and rs.shape == (n, 16)
        assert ex.shape == (3 * n,) and rc.shape == (64,) and rpe.shape == (8,) and rpe.dtype == torch.int64
        y = torch.empty(500, 2048, dtype=torch.bfloat16, device="cuda")
        assert lib.moe_combine_prefill(y, ids, w, ex, rc, "ep", 0, 8).shape == (100, 2048)
        npr = torch.empty(8, dtype=torch.int32, device="cuda")
        a, b, c, d = lib.notify_dispatch(npe, npr, "ep", 8, 2048, 100)
        assert a.shape == (64,) and b.shape == (64,) and c.shape == (8,) and d.shape == (4,)
    with pytest.raises(RuntimeError):
        with FakeTensorMode():
            lib.get_dispatch_layout(torch.empty(4, 2, dtype=torch.int64), 7, 2)   # 7 experts over 2 ranks


@pytest.mark.skipif(not ops.CPP_LIBRARY_LOADED, reason="C++ operator library not built")
def test_torch_compile_traces_a_module_that_calls_fused_deep_moe():
    """fullgraph=True: the operator must not break the graph. The backend only inspects the captured graph (the
    kernels need a GPU); what is checked is that tracing goes through the Meta function."""
    seen = {}

    def backend(gm, example_inputs):
        seen["targets"] = [str(n.target) for n in gm.graph.nodes if n.op == "call_function"]
        return lambda *a: (torch.zeros(64, 1024),)

    class Layer(torch.nn.Module):
        def forward(self, x, ids, scales, w1, s1, w2, s2):
            out, share, _ = lib.fused_deep_moe(x, ids, [w1], [s1], [w2], [s2], scales, None, None, None, None, None,
                                               None, None, "ep", 2, 0, 8, 0, 128)
            return out + share

    a = _moe_args()
    torch.compile(Layer(), backend=backend, fullgraph=True)(a[0], a[1], a[6], a[2][0], a[3][0], a[4][0], a[5][0])
    assert any("fused_deep_moe" in t for t in seen["targets"]), seen


@pytest.mark.skipif(not ops.CPP_LIBRARY_LOADED, reason="C++ operator library not built")
def test_operators_are_marked_not_differentiable():
    ids = torch.randint(0, 8, (16, 2))
    npe, _ = lib.get_dispatch_layout(ids, 8, 2)
    assert int(npe.sum()) == 32
    x = torch.randn(16, 128, requires_grad=True)
    y = lib.moe_combine_prefill(x, ids, torch.rand(16, 2), torch.zeros(48, dtype=torch.int32),
                                torch.zeros(8, dtype=torch.int32), "solo", 0, 1)
    with pytest.raises(RuntimeError, match="not implemented|does not require grad|derivative"):
        y.sum().backward()


def test_weight_lists_are_viewed_or_stacked_once():
    w = torch.randn(6, 8, 4)
    views = list(w.unbind(0))
    st = ops._as_stacked(views)
    assert st.data_ptr() == w.data_ptr() and torch.equal(st, w)          # contiguous pieces: no copy at all
    parts = [torch.randn(8, 4) for _ in range(6)]
    a = ops._as_stacked(parts)
    assert ops._as_stacked(parts) is a and torch.equal(a, torch.stack(parts))   # stacked once, then reused
    parts[2].add_(1.0)                                                   # an in-place update invalidates the copy
    b = ops._as_stacked(parts)
    assert b is not a and torch.equal(b, torch.stack(parts))
    f8 = [torch.randint(0, 255, (8, 4), dtype=torch.uint8).view(torch.float8_e4m3fn) for _ in range(3)]
    assert ops._as_stacked(f8).dtype == torch.float8_e4m3fn and ops._as_stacked(f8).shape == (3, 8, 4)
    single = torch.randn(3, 8, 4)
    assert ops._as_stacked([single]) is single


def test_smooth_scales_move_into_the_gate_up_weights():
    from umdk_b200.ops.ep_ll import ExpertWeights
    g = torch.Generator().manual_seed(0)
    G, F, H = 2, 128, 256
    w1q, w1s = ref.quant_fp8_128x128(torch.randn(G, 2 * F, H, generator=g) * 0.05)
    w2q, w2s = ref.quant_fp8_128x128(torch.randn(G, H, F, generator=g) * 0.05)
    w = ExpertWeights(w1q, w1s, w2q, w2s)
    smooth = 0.5 + torch.rand(G, H, generator=g)
    f = ops._fold_smooth(w, smooth)
    assert ops._fold_smooth(w, smooth) is f and f.w2q is w.w2q
    x = torch.randn(5, H, generator=g)
    for e in range(G):
        want = (x * smooth[e]) @ ref.dequant_fp8_128x128(w1q[e], w1s[e]).t()
        got = x @ ref.dequant_fp8_128x128(f.w1q[e], f.w1s[e]).t()
        assert ref.mean_rel_err(got, want) < 0.05
