"""Flagship decoder: the offloaded-KV path must give the same tokens as the all-resident path, and the MoE block of
a layer must match the dense fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, cfg.vocab, (cfg.batch,), generator=g).cuda()
    idx = [torch.stack([torch.randperm(cfg.ctx + 1, generator=g)[:cfg.topk_kv] for _ in range(cfg.batch)])
           .to(torch.int32).cuda() for _ in range(cfg.n_layers)]
    return tokens, idx


def test_offloaded_kv_matches_resident_kv():
    from umdk_b200.models.dsv3_decoder import DecoderConfig, DecoderRank
    outs = []
    for offload in (True, False):
        cfg = DecoderConfig.tiny()
        cfg.offload = offload
        m = DecoderRank(cfg)
        tokens, idx = _inputs(cfg)
        if offload:
            # scribble over the staging pages: only a working prefetch can restore them
            for pool in m.kv:
                pool[m.n_resident:].zero_()
        for _ in range(3):
            nxt = m.step(tokens, idx)
        torch.cuda.synchronize()
        m.check()
        if offload:
            assert m.kvm.stats()["bytes_h2d"] == 3 * cfg.n_layers * m.n_staging * 64 * 576 * 2
        outs.append(nxt.cpu())
        m.close()
    assert torch.equal(outs[0], outs[1])


def test_decoder_moe_block_matches_oracle():
    from umdk_b200.models.dsv3_decoder import DecoderConfig, DecoderRank, reference_layer_moe
    from umdk_b200.ops import reference as ref
    cfg = DecoderConfig.tiny()
    cfg.offload = False
    m = DecoderRank(cfg)
    g = torch.Generator().manual_seed(3)
    h = torch.randn(cfg.batch, cfg.hidden, generator=g).to(torch.bfloat16).cuda()
    L = m.layers[0]
    probs = torch.softmax(h.float() @ L["router"].t(), dim=-1)
    w, idx = torch.topk(probs, cfg.top_k, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).contiguous()
    out, share, cnt = m.ep.moe(h, idx.contiguous(), w, L["experts"], L["shared"])
    torch.cuda.synchronize()
    m.check()
    want = reference_layer_moe(cfg, h.cpu(), idx.cpu(), w.cpu(), L["experts"])
    assert ref.mean_rel_err(out.float().cpu(), want) < 0.02
    assert int(cnt.sum()) == cfg.batch * cfg.top_k
    m.close()
