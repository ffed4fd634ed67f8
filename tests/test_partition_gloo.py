"""CPU tests of the multi-GPU host logic: world-size-2 (and 3) `gloo` process
groups run the same partition/broadcast plan that bench.py runs over NCCL,
with numpy standing in for the GPU kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from polygeist_b200 import partition


def test_row_blocks_cover_and_align():
    for M, P in [(4096, 8), (1000, 3), (128, 4), (5, 2)]:
        b = partition.row_blocks(M, P, align=128)
        assert b[0] == 0 and b[-1] == M and len(b) == P + 1
        assert all(x <= y for x, y in zip(b, b[1:]))
        assert all(x % 128 == 0 for x in b[1:-1])


def test_syrk_blocks_balance_area():
    N, P = 16384, 8
    b = partition.syrk_row_blocks(N, P, align=128)
    area = [(b[p + 1] * (b[p + 1] + 1) - b[p] * (b[p] + 1)) / 2 for p in range(P)]
    assert b[0] == 0 and b[-1] == N
    assert max(area) / min(area) < 1.16          # equal heights would give 15x
    eq = partition.row_blocks(N, P, align=128)
    area_eq = [(eq[p + 1] * (eq[p + 1] + 1) - eq[p] * (eq[p] + 1)) / 2 for p in range(P)]
    assert max(area_eq) / min(area_eq) > 10


def test_slice_groups():
    assert partition.slice_groups(16) == [(0, 1), (1, 2), (2, 4), (4, 8), (8, 16)]
    assert partition.slice_groups(5) == [(0, 1), (1, 2), (2, 4), (4, 5)]
    assert partition.slice_groups(1) == [(0, 1)]
    assert partition.slice_groups(0) == []
    assert partition.slice_groups(3, grow=False) == [(0, 1), (1, 2), (2, 3)]
    for n in range(1, 40):       # a partition of range(n), in order
        g = partition.slice_groups(n)
        assert g[0][0] == 0 and g[-1][1] == n and all(a[1] == b[0] for a, b in zip(g, g[1:]))


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_pull_schedule_delivers_every_slice_without_deadlock(world):
    """All ranks' copy-stream lists run against each other: a wait blocks until
    the owner has signalled, a pull may only read rows its source already
    holds, and when a slice is declared ready all its rows are there."""
    chunks = [(0, 5), (5, 16), (16, 17), (17, 64)]
    for src in (0, world - 1):
        ops = {r: partition.pull_schedule(r, world, src, chunks) for r in range(world)}
        pc = {r: 0 for r in range(world)}
        signalled, have = set(), {r: set() for r in range(world)}
        have[src] = set(range(chunks[-1][1]))
        progress = True
        while progress:
            progress = False
            for r in range(world):
                while pc[r] < len(ops[r]):
                    op = ops[r][pc[r]]
                    if op[0] == "wait" and (op[1], op[2]) not in signalled:
                        break
                    if op[0] == "pull":
                        rows = set(range(op[2], op[3]))
                        assert rows <= have[op[1]], (r, op)
                        have[r] |= rows
                    elif op[0] == "signal":
                        signalled.add((r, op[1]))
                    elif op[0] == "ready":
                        k0, k1 = chunks[op[1]]
                        assert set(range(k0, k1)) <= have[r]
                    pc[r] += 1
                    progress = True
        assert all(pc[r] == len(ops[r]) for r in range(world)), "deadlock"
        assert [op[1] for op in ops[src] if op[0] == "ready"] == list(range(len(chunks)))


def test_k_chunks():
    assert partition.k_chunks(10, 4) == [(0, 4), (4, 8), (8, 10)]
    assert partition.k_chunks(0, 4) == [(0, 0)]
    assert partition.k_chunks(10, 10, first=2) == [(0, 2), (2, 10)]
    assert partition.k_chunks(10, 4, first=3) == [(0, 3), (3, 7), (7, 10)]
    assert partition.k_chunks(10, 4, first=10) == partition.k_chunks(10, 4)   # no room for a head


def test_pull_plan_covers_every_row_once():
    for world, src in [(2, 0), (3, 1), (8, 0)]:
        k0, k1 = 100, 100 + 37 * world
        for rank in range(world):
            p1, p2 = partition.pull_plan(rank, world, src, k0, k1)
            if rank == src:
                assert p1 == [] and p2 == []
                continue
            got = sorted((r0, r1) for _, r0, r1 in p1 + p2)
            assert got[0][0] == k0 and got[-1][1] == k1
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))       # contiguous, no overlap
            assert all(peer == src for peer, _, _ in p1)                  # own piece straight from the source
            assert all(peer not in (src, rank) for peer, _, _ in p2)      # the rest from its owners
        # the source sends each row exactly once in phase 1
        sent = sorted((r0, r1) for rank in range(world) if rank != src
                      for _, r0, r1 in partition.pull_plan(rank, world, src, k0, k1)[0])
        assert sent[0][0] == k0 and sent[-1][1] == k1 and all(a[1] == b[0] for a, b in zip(sent, sent[1:]))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _np_gemm(alpha, A, B, beta, C):
    C.copy_(torch.from_numpy(alpha * (A.numpy() @ B.numpy()) + beta * C.numpy()))


def _np_syrk(alpha, A, beta, Cb, rows):
    r0, r1 = rows
    full = alpha * (A.numpy()[r0:r1] @ A.numpy().T) + beta * Cb.numpy()[:, :r1]
    out = Cb.numpy()
    for i in range(r1 - r0):
        out[i, : r0 + i + 1] = full[i, : r0 + i + 1]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)
        M, N, K = 96, 40, 64
        A = rng.uniform(-1, 1, (M, K))
        B = rng.uniform(-1, 1, (K, N))
        C = rng.uniform(-1, 1, (M, N))
        ref = 1.5 * A @ B + 1.2 * C
        b = partition.row_blocks(M, world, align=16)
        r0, r1 = b[rank], b[rank + 1]
        A_p = torch.from_numpy(A[r0:r1].copy())
        C_p = torch.from_numpy(C[r0:r1].copy())
        B_local = torch.from_numpy(B.copy()) if rank == 0 else torch.full((K, N), float("nan"), dtype=torch.float64)
        plan = partition.PartitionedGemm(dist, _np_gemm, src=0, chunk=24)
        plan.run(1.5, A_p, B_local, 1.2, C_p)
        ok = np.allclose(C_p.numpy(), ref[r0:r1], rtol=1e-13, atol=1e-13)
        ok = ok and np.array_equal(B_local.numpy(), B)       # every rank ends with all of B
        # a narrow first K-slice, then the rest in one piece
        C_q = torch.from_numpy(C[r0:r1].copy())
        B_q = torch.from_numpy(B.copy()) if rank == 0 else torch.full((K, N), float("nan"), dtype=torch.float64)
        partition.PartitionedGemm(dist, _np_gemm, src=0, chunk=K, first_chunk=8).run(1.5, A_p, B_q, 1.2, C_q)
        ok = ok and np.allclose(C_q.numpy(), ref[r0:r1], rtol=1e-13, atol=1e-13)
        ok = ok and np.array_equal(B_q.numpy(), B)

        Ns, Ks = 80, 24
        As = rng.uniform(0, 1, (Ns, Ks))
        Cs = rng.uniform(0, 1, (Ns, Ns))
        refs = np.where(np.tril(np.ones((Ns, Ns), bool)), 1.5 * As @ As.T + 1.2 * Cs, Cs)
        sp = partition.PartitionedSyrk(dist, _np_syrk, src=0, kchunk=10, align=8)
        bs = sp.blocks(Ns)
        s0, s1 = bs[rank], bs[rank + 1]
        A_loc = torch.from_numpy(As.copy()) if rank == 0 else torch.full((Ns, Ks), float("nan"), dtype=torch.float64)
        C_blk = torch.from_numpy(Cs[s0:s1].copy())
        sp.run(1.5, A_loc, 1.2, C_blk)
        ok = ok and np.allclose(C_blk.numpy(), refs[s0:s1], rtol=1e-13, atol=1e-13)
        # The same plan object with another N but the same number of K-slices:
        # its packed-slice buffers must be rebuilt, not reused.
        N2 = 56
        A2 = rng.uniform(0, 1, (N2, Ks))
        C2 = rng.uniform(0, 1, (N2, N2))
        ref2 = np.where(np.tril(np.ones((N2, N2), bool)), 1.5 * A2 @ A2.T + 1.2 * C2, C2)
        b2 = sp.blocks(N2)
        t0, t1 = b2[rank], b2[rank + 1]
        A2_loc = torch.from_numpy(A2.copy()) if rank == 0 else torch.full((N2, Ks), float("nan"), dtype=torch.float64)
        C2_blk = torch.from_numpy(C2[t0:t1].copy())
        sp.run(1.5, A2_loc, 1.2, C2_blk)
        ok = ok and np.allclose(C2_blk.numpy(), ref2[t0:t1], rtol=1e-13, atol=1e-13)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_partitioned_plans_over_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(res) == [(r, True) for r in range(world)]
