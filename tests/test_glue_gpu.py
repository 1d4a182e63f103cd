"""The fused glue kernels of the decode step, each against the chain of plain torch ops it replaces."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rope(x, cos, sin):
    x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2).to(x.dtype)


def _close(a, b, tol=1.5e-2):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() <= tol * b.abs().max()).item() and ((a - b).norm() / b.norm()).item() < 4e-3


@pytest.mark.parametrize("T,H", [(64, 7168), (8, 1024), (3, 8192), (5, 136)])
def test_add_rmsnorm(T, H):
    from umdk_b200.ops import glue
    g = torch.Generator(device="cuda").manual_seed(T + H)
    x = (torch.randn(T, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    a = (torch.randn(T, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn(T, H, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    x0, h0 = glue.add_rmsnorm(x, w)
    assert x0 is x and _close(h0, F.rms_norm(x, (H,), w))
    x1, h1 = glue.add_rmsnorm(x, w, a, b)
    want_x = (x.float() + a.float() + b.float()).to(torch.bfloat16)
    assert torch.equal(x1, want_x) and _close(h1, F.rms_norm(want_x, (H,), w))
    x2, h2 = glue.add_rmsnorm(x, w, a)
    assert torch.equal(x2, (x.float() + a.float()).to(torch.bfloat16))
    # a strided input (rows of a wider matrix)
    wide = (torch.randn(T, H + 64, device="cuda", generator=g)).to(torch.bfloat16)
    _, h3 = glue.add_rmsnorm(wide[:, :H], w)
    assert _close(h3, F.rms_norm(wide[:, :H], (H,), w))


def test_qkv_post_and_q_rope():
    from umdk_b200.ops import glue
    g = torch.Generator(device="cuda").manual_seed(1)
    T, q_lora, heads, nope = 16, 1536, 128, 128
    qkv = torch.randn(T, q_lora + 576, device="cuda", generator=g).to(torch.bfloat16)
    qn = (1 + 0.1 * torch.randn(q_lora, device="cuda", generator=g)).to(torch.bfloat16)
    kn = (1 + 0.1 * torch.randn(512, device="cuda", generator=g)).to(torch.bfloat16)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, device="cuda", dtype=torch.float32) / 64))
    cos, sin = torch.cos(777.0 * inv_freq), torch.sin(777.0 * inv_freq)
    pool = torch.zeros(40, 64, 576, device="cuda", dtype=torch.bfloat16)
    new_row = (torch.randperm(40, device="cuda", generator=g)[:T] * 64 + 5).to(torch.int64)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    qa = glue.qkv_post(qkv, q_lora, qn, kn, cos, sin, pool, new_row, status)
    assert status.tolist()[0] == 0
    assert _close(qa, F.rms_norm(qkv[:, :q_lora], (q_lora,), qn))
    want_row = torch.cat((F.rms_norm(qkv[:, q_lora:q_lora + 512], (512,), kn), _rope(qkv[:, q_lora + 512:], cos, sin)), -1)
    got_row = pool.view(-1, 576)[new_row]
    assert _close(got_row, want_row)
    assert int((pool.view(-1, 576).abs().sum(-1) > 0).sum()) == T      # nothing else was written
    # a row outside the pool is refused with a status, not written
    bad = new_row.clone()
    bad[3] = 40 * 64
    glue.qkv_post(qkv, q_lora, qn, kn, cos, sin, pool, bad, status)
    assert status.tolist()[0] == 3
    q = torch.randn(T, heads, nope + 64, device="cuda", generator=g).to(torch.bfloat16)
    q_full = torch.zeros(T, heads, 576, device="cuda", dtype=torch.bfloat16)
    glue.q_rope(q, nope, cos, sin, q_full)
    assert _close(q_full[..., 512:], _rope(q[..., nope:], cos, sin)) and float(q_full[..., :512].abs().sum()) == 0.0


@pytest.mark.parametrize("E,K", [(256, 8), (16, 4), (1024, 6), (40, 3)])
def test_router_topk(E, K):
    from umdk_b200.ops import glue
    g = torch.Generator(device="cuda").manual_seed(E)
    logits = torch.randn(33, E, device="cuda", generator=g).to(torch.bfloat16)
    idx, w = glue.router_topk(logits, K)
    pw, pidx = torch.topk(torch.softmax(logits.float(), -1), K, dim=-1)
    # bf16 logits can tie: compare the selected VALUES, and ids where values are distinct
    assert torch.allclose(torch.gather(logits.float(), 1, idx), torch.gather(logits.float(), 1, pidx))
    assert torch.allclose(w, pw / pw.sum(-1, keepdim=True), atol=1e-5)
    assert all(len(set(r)) == K for r in idx.tolist())
