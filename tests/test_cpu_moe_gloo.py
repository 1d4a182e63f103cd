"""CPU / gloo world_size=2 check of the MoE operator contract: 128 tokens per rank, hidden 1024, fp32 activations
N(0,1), 16 experts (8 per rank), top-2 routing from softmax of N(0,1) gate logits with renormalised weights, expert
k = identity * (k + 1); combine(dispatch(x)) must equal the dense reference."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from umdk_b200.ops import reference as ref


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs(rank, T=128, H=1024, E=16, K=2):
    g = torch.Generator().manual_seed(0 + rank)
    x = torch.randn(T, H, generator=g)
    p = torch.softmax(torch.randn(T, E, generator=g), dim=-1)
    w, idx = torch.topk(p, K, dim=-1)
    return x, idx.to(torch.int64), (w / w.sum(-1, keepdim=True)).float()


def _worker(rank, world, port, use_ops, quant, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        E = 16
        x, idx, w = _inputs(rank)
        el = E // world
        if use_ops:
            import umdk_b200
            ops = umdk_b200.load_torch_ops()
            ops.register_group("ep", None)
            o = torch.ops.umdk_cam_op_lib
            npe, sidx = o.get_dispatch_layout(idx, E, world)
            recv_x, scales, expand_idx, recv_count, per_expert = o.moe_dispatch_prefill(
                x, idx, w, npe, sidx, "ep", rank, world, quant)
            npr = ref.ref_layout(idx, E, world).num_tokens_per_rank
            n_cnt, n_off, n_pe, n_tot = o.notify_dispatch(npe, npr, "ep", idx.shape[1], x.shape[1], x.shape[0])
            assert torch.equal(n_cnt, recv_count) and torch.equal(n_pe, per_expert)
            assert n_tot[0] == recv_x.shape[0] and torch.equal(n_off[1:], n_cnt[:-1])
            xin = ref.dequant_fp8_1x128(recv_x, scales) if quant else recv_x
            le = torch.repeat_interleave(torch.arange(el), per_expert)
            y = xin * (le + rank * el + 1).float().unsqueeze(1)
            out = o.moe_combine_prefill(y, idx, w, expand_idx, recv_count, "ep", rank, world)
        else:
            from umdk_b200 import Buffer
            buf = Buffer(None)
            _, _, npe, in_rank, _ = buf.get_dispatch_layout(idx, E)
            recv_x, recv_le, recv_w, per_expert, handle, _ = buf.dispatch(
                x, topk_idx=idx, topk_weights=w, num_tokens_per_expert=npe, use_fp8=quant)
            xin = ref.dequant_fp8_1x128(*recv_x) if quant else recv_x
            assert sum(per_expert) == xin.shape[0] == recv_le.numel()
            y = xin * (recv_le + rank * el + 1).float().unsqueeze(1)
            out, _, _ = buf.combine(y, handle)
        xr = ref.dequant_fp8_1x128(*ref.quant_fp8_1x128(x)) if quant else x
        dense = ref.dense_moe_reference(xr, idx, w, lambda e, v: v * (e + 1))
        err = ref.mean_rel_err(out.float(), dense)
        q.put((rank, err))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # surface the failure in the parent
        import traceback
        q.put((rank, "ERR " + traceback.format_exc()))


@pytest.mark.parametrize("use_ops,quant", [(False, False), (True, False), (False, True), (True, True)])
def test_combine_of_dispatch_matches_dense_reference(use_ops, quant):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, use_ops, quant, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, err in res:
        assert not isinstance(err, str), err
        assert err < (5e-3 if quant else 1e-5), (rank, err)
