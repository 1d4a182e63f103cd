"""Sparse MLA decode kernel against the fp32 PyTorch statement of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, ctx, topk, seed, frac_invalid=0.0):
    from umdk_b200.ops.attention import DIM, HEADS, PAGE
    g = torch.Generator().manual_seed(seed)
    pages_per_seq = (ctx + PAGE - 1) // PAGE
    num_pages = B * pages_per_seq + 3
    kv = (torch.randn(num_pages, PAGE, DIM, generator=g) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(num_pages, generator=g)[:B * pages_per_seq]
    bt = perm.reshape(B, pages_per_seq).to(torch.int32)
    q = (torch.randn(B, HEADS, DIM, generator=g) * 0.5).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(ctx, generator=g)[:topk] for _ in range(B)]).to(torch.int32)
    if frac_invalid > 0:
        m = torch.rand(B, topk, generator=g) < frac_invalid
        idx[m] = -1
    return q, kv, bt, idx


@pytest.mark.parametrize("B,ctx,topk,splits,inv", [
    (1, 64, 64, 1, 0.0),
    (2, 512, 128, 1, 0.1),
    (3, 1000, 200, 1, 0.3),
    (2, 4096, 512, 2, 0.0),
    (4, 8192, 2048, 1, 0.0),
    (2, 8192, 2048, 4, 0.05),
    (2, 32768, 2048, 1, 0.0),      # the serving benchmark's context and key count
    (1, 8192, 4096, 1, 0.02),      # more keys than one CTA pair resolves: the wrapper raises the split count
    (3, 300, 50, 3, 0.0),          # splits with no keys at all
])
def test_sparse_mla_decode(B, ctx, topk, splits, inv):
    from umdk_b200.ops.attention import ref_sparse_mla_decode, sparse_mla_decode
    q, kv, bt, idx = _case(B, ctx, topk, seed=B * 7 + topk, frac_invalid=inv)
    scale = 576 ** -0.5
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out, lse = sparse_mla_decode(q.cuda(), kv.cuda(), bt.cuda(), idx.cuda(), scale, num_splits=splits, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    want, want_lse = ref_sparse_mla_decode(q, kv, bt, idx, scale)
    err = (out.float().cpu() - want).abs().max().item()
    rel = ((out.float().cpu() - want).norm() / want.norm()).item()
    assert rel < 2e-2, (err, rel)
    assert torch.allclose(lse.cpu(), want_lse, atol=2e-2, rtol=1e-3)
