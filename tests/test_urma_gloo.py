"""URMA semantics over the shared-memory provider with two gloo ranks (separate processes): each rank registers a
1 MiB fp32 segment, writes 4096 random fp32 N(0,1) values into the peer's segment with a one-sided write, reads them
back with a one-sided read (bit exact), and both ranks perform 10 000 fetch-add increments on an int64 counter owned
by rank 0 (exact sum). Also two-sided send/recv with immediate data, CAS, access control and timeouts."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, shm_dir, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["URMA_SHM_DIR"] = shm_dir
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from umdk_b200 import urma
        ctx = urma.Context("shm0")
        ep = ctx.endpoint(depth=512, recv_token=11)
        seg_mem = torch.zeros(1 << 18, dtype=torch.float32)           # 1 MiB
        counter = torch.zeros(8, dtype=torch.int64)
        seg = ctx.register(seg_mem, token=100 + rank)
        cseg = ctx.register(counter, token=7)
        ro_mem = torch.arange(16, dtype=torch.int64)
        ro = ctx.register(ro_mem, access=urma.READ, token=5)
        blobs = [None] * world
        dist.all_gather_object(blobs, (ep.blob, seg.blob, cseg.blob, ro.blob))
        peer_rank = 1 - rank
        peer = ctx.import_endpoint(blobs[peer_rank][0], token=11)
        rseg = ctx.import_segment(blobs[peer_rank][1], token=100 + peer_rank)
        rcnt = ctx.import_segment(blobs[0][2], token=7)
        owner0 = ctx.import_endpoint(blobs[0][0], token=11)
        # one-sided write of 4096 values into the peer's segment at an offset, then read them back
        g = torch.Generator().manual_seed(rank)
        src = torch.randn(4096, generator=g)
        off = 4096 * 4 * (rank + 1)
        ep.write(peer, rseg, rseg.va + off, src.data_ptr(), src.numel() * 4)
        ep.wait(1)
        back = torch.zeros(4096)
        ep.read(peer, rseg, rseg.va + off, back.data_ptr(), back.numel() * 4)
        ep.wait(1)
        assert torch.equal(back, src), "read-back differs from what was written"
        dist.barrier()
        # the peer's write landed in my memory
        gp = torch.Generator().manual_seed(peer_rank)
        want = torch.randn(4096, generator=gp)
        poff = 4096 * (peer_rank + 1)
        assert torch.equal(seg_mem[poff:poff + 4096], want)
        # 10k fetch-adds per rank on rank 0's counter, pipelined 64 deep
        n_ops, depth, done, posted = 10000, 64, 0, 0
        while done < n_ops:
            while posted < n_ops and posted - done < depth:
                ep.atomic(owner0, urma.OPC_FADD, rcnt, rcnt.va, 1)
                posted += 1
            done += len(ep.wait(1, check=True))
            done += len(ep.poll(64))
        dist.barrier()
        if rank == 0:
            assert int(counter[0]) == world * n_ops, int(counter[0])
        # compare-and-swap: exactly one rank wins
        old = ep.compare_swap(owner0, rcnt, rcnt.va + 8, 0, rank + 1)
        wins = [None] * world
        dist.all_gather_object(wins, old == 0)
        assert sum(wins) == 1
        # two-sided send with immediate data
        rbuf = torch.zeros(64, dtype=torch.float32)
        ep.post_recv(rbuf, user_ctx=99)
        dist.barrier()
        msg = torch.full((64,), float(rank + 1))
        ep.send(peer, msg.data_ptr(), 256, user_ctx=5, imm=1000 + rank)
        cs = ep.wait(2)
        rc = [c for c in cs if c.is_recv][0]
        assert rc.user_ctx == 99 and rc.length == 256 and rc.imm == 1000 + peer_rank
        assert torch.equal(rbuf, torch.full((64,), float(peer_rank + 1)))
        # access control: a write into a read-only segment and a wrong token both complete with an error status
        rro = ctx.import_segment(blobs[peer_rank][3], token=5)
        ep2 = ctx.endpoint(depth=16, recv_token=11)
        ep2.write(peer, rro, rro.va, src.data_ptr(), 8)
        c = ep2.wait(1, check=False)
        assert len(c) == 1 and c[0].status == urma.CR_REM_ACCESS_ABORT
        bad = ctx.import_segment(blobs[peer_rank][1], token=424242)
        ep3 = ctx.endpoint(depth=16, recv_token=11)
        ep3.read(peer, bad, bad.va, back.data_ptr(), 8)
        c = ep3.wait(1, check=False)
        assert len(c) == 1 and c[0].status == urma.CR_REM_ACCESS_ABORT
        # invalid access combination is refused at registration (WRITE without READ)
        try:
            ctx.register(torch.zeros(4), access=urma.WRITE)
            raise AssertionError("WRITE-only registration must fail")
        except urma.UrmaError:
            pass
        dist.barrier()
        ctx.close()
        q.put((rank, "ok"))
        dist.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, "ERR " + traceback.format_exc()))


def test_urma_two_ranks(tmp_path):
    world = 2
    mpctx = mp.get_context("spawn")
    q = mpctx.Queue()
    port = _free_port()
    procs = [mpctx.Process(target=_worker, args=(r, world, port, str(tmp_path), q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in res:
        assert msg == "ok", msg
