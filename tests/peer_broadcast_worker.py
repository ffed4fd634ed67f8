"""One rank of the copy-engine broadcast check (launched by
test_gpu_runtime.py::test_peer_pull_broadcast_matches_nccl through torchrun).

Every rank owns a row block of C = alpha*A*B + beta*C; B lives on rank 0 and
travels in K-slices, once by the NCCL broadcast and once by PeerPullBroadcast
(copy engines over peer-mapped symmetric memory, stream-ordered signals
between the two pull phases when there are more than two ranks).  Both routes
must leave the same bits in B on every rank and in C."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import polygeist_b200 as pgb  # noqa: E402
from polygeist_b200 import partition  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import torch.distributed._symmetric_memory as symm_mem

    M, N, K, chunk = 1024 * world, 1536, 4096, 256       # 16 slices, ragged pieces for 3 ranks
    b = partition.row_blocks(M, world)
    r0, r1 = b[rank], b[rank + 1]

    def filled(rows, cols, aid, row0=0):
        t = torch.empty((rows, cols), dtype=torch.float32, device=dev)
        pgb.fill_uniform(t, 7, aid, 0.0, 1.0, row0=row0)
        return t

    A, C0 = filled(r1 - r0, K, 1, r0), filled(r1 - r0, N, 3, r0)
    buf = symm_mem.empty((K, N), dtype=torch.float32, device=dev)
    hb = symm_mem.rendezvous(buf, dist.group.WORLD)
    views = [hb.get_buffer(r, (K, N), torch.float32) for r in range(world)]
    flags = memops = None
    if world > 2:
        fl = symm_mem.empty((world, 64), dtype=torch.int32, device=dev)
        fl.zero_()
        hf = symm_mem.rendezvous(fl, dist.group.WORLD)
        flags = [hf.get_buffer(r, (world, 64), torch.int32) for r in range(world)]
        memops = partition.stream_memops()
    peer = partition.PeerPullBroadcast(torch, dist, views, src=0, flags=flags, memops=memops)
    B = views[rank]
    results = {}
    for route in ("nccl", "peer", "peer"):                # the second peer run reuses the flag words
        if rank == 0:
            pgb.fill_uniform(B, 7, 2, 0.0, 1.0)
        else:
            B.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        plan = partition.PartitionedGemm(dist, pgb.gemm, src=0, chunk=chunk,
                                         peer_broadcast=peer if route == "peer" else None)
        Cm = C0.clone()
        plan.run(1.5, A, B, 1.2, Cm)
        torch.cuda.synchronize()
        pgb.poll_device_status()
        assert not bool(torch.isnan(B).any()), f"rank {rank}: rows of B missing ({route})"
        key = route + str(len(results))
        results[key] = (B.clone(), Cm)
    ref_b, ref_c = results["nccl0"]
    for key, (gb, gc) in results.items():
        assert torch.equal(gb, ref_b), f"rank {rank}: B differs ({key})"
        assert torch.equal(gc, ref_c), f"rank {rank}: C differs ({key})"
    # the operand really is the source's: compare with rank 0's generator output
    want = torch.empty((K, N), dtype=torch.float32, device=dev)
    pgb.fill_uniform(want, 7, 2, 0.0, 1.0)
    assert torch.equal(ref_b, want)
    dist.barrier()
    if rank == 0:
        print("PEER_BROADCAST_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
