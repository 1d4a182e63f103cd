"""Two or more GPU ranks run all-reduce steps on plain peer loads (no NVLS); the last rank leaves between two steps,
announcing it through the membership view; the others see that on the host BEFORE launching the next step, skip the
launch, and finish with a clean kernel status. No kernel is ever launched against the departed rank."""
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()),
                            timeout=datetime.timedelta(seconds=60))
    from umdk_b200.ops.tp import AllReduce
    from umdk_b200.parallel.membership import Membership
    from umdk_b200.parallel.symm import SymmetricHeap
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=60))
    member = Membership(store, rank, world, timeout_s=5.0)
    assert member.wait_for_all(30)
    n = 1 << 16
    heap = SymmetricHeap(AllReduce.heap_bytes(n * 2, world))
    ar = AllReduce(heap, n * 2)
    leaver = world - 1
    done_steps = 0
    for step in range(6):
        member.beat()
        if rank == leaver and step == 3:
            torch.cuda.synchronize()            # nothing of this rank is in flight
            member.leave()
            break
        if rank != leaver and step >= 3:
            # give the announcement time to arrive, then look before launching anything
            deadline = time.time() + 20
            while leaver in member.alive() and time.time() < deadline:
                time.sleep(0.01)
        if member.departed():
            break                               # a peer is gone: do not launch against it
        x = torch.full((n,), float(rank + 1 + step), dtype=torch.bfloat16, device="cuda")
        out = ar(x, algo="one_shot")            # peer loads, not multimem
        torch.cuda.synchronize()
        ar.check()
        want = sum(r + 1 + step for r in range(world))
        assert torch.allclose(out.float(), torch.full((n,), float(want), device="cuda"))
        done_steps += 1
    assert done_steps == 3, done_steps
    ar.check()                                  # survivors: no timeout recorded, the context is healthy
    y = torch.ones(8, device="cuda") * 2
    assert float(y.sum()) == 16.0
    if rank != leaver:
        assert member.departed() == [leaver]
    print(f"MP_LEAVE_OK rank {rank}", flush=True)
    if rank == 0:
        time.sleep(1.0)                         # keep the store up while the others finish
    # no collective teardown: the group has lost a member; every rank simply ends
    os._exit(0)


if __name__ == "__main__":
    main()
