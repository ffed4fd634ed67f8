"""Row-block partitioning of a contraction over the GPUs of one box.

One process per GPU (`torch.distributed`).  Rank p owns a block of rows of the
output and of the left operand; the shared right operand lives on one rank and
is broadcast K-chunk by K-chunk while the chunks already received are being
multiplied, so only the first chunk's transfer is exposed.  The reference has
no multi-GPU path; this module is the host-side plan for the partition named
by the raised-contraction design (rows are independent in the loop nests,
gemm.c:104-113, syrk.c:97-106, which is what makes the split exact).

The scheduling logic is backend-agnostic: with `gloo` and CPU tensors plus a
caller-supplied `compute` it runs without a GPU (that is how it is tested).
"""
import math


def row_blocks(M, P, align=128):
    """Equal-height row blocks [b[p], b[p+1]) with boundaries on `align`."""
    if P <= 0:
        raise ValueError("P must be positive")
    b = [0]
    for p in range(1, P):
        x = (M * p) // P
        x = min(M, (x + align // 2) // align * align) if align > 1 else x
        b.append(max(x, b[-1]))
    b.append(M)
    return b


def syrk_row_blocks(N, P, align=128):
    """Row blocks of a lower-triangular update with equal *areas*: row i costs
    i+1 outputs, so the boundaries sit at N*sqrt(p/P) rather than N*p/P
    (equal heights would give the last rank (2P-1)x the work of the first)."""
    b = [0]
    for p in range(1, P):
        x = int(round(N * math.sqrt(p / P)))
        x = min(N, (x + align // 2) // align * align) if align > 1 else x
        b.append(max(x, b[-1]))
    b.append(N)
    return b


def k_chunks(K, chunk, first=0):
    """[k0,k1) slices of the inner extent: `chunk` wide, optionally preceded by
    one narrower slice of `first` (so the first product can start while most
    of the shared operand is still in flight)."""
    chunk = max(1, int(chunk))
    first = min(int(first), K)
    head = [(0, first)] if 0 < first < K else []
    start = first if head else 0
    return head + [(k0, min(K, k0 + chunk)) for k0 in range(start, K, chunk)] or [(0, 0)]


def pull_plan(rank, world, src, k0, k1):
    """Copy-engine broadcast of rows [k0,k1) from `src`, as pulls by `rank`.

    Returns (phase1, phase2): lists of (peer, r0, r1) meaning "copy rows
    [r0,r1) from `peer`'s buffer into mine".  The rows are split into world-1
    pieces, one per non-source rank.  Phase 1: every non-source rank pulls its
    own piece from `src` (so `src` sends each row once).  Phase 2 (after all
    ranks finished phase 1): it pulls every other piece from the rank that
    owns it, so the remaining traffic is spread over all links.
    """
    others = [r for r in range(world) if r != src]
    if rank == src or not others:
        return [], []
    n = len(others)
    rows = k1 - k0
    bounds = [k0 + (rows * j) // n for j in range(n + 1)]
    piece = {r: (bounds[j], bounds[j + 1]) for j, r in enumerate(others)}
    p1 = [(src,) + piece[rank]] if piece[rank][1] > piece[rank][0] else []
    p2 = [(q,) + piece[q] for q in others if q != rank and piece[q][1] > piece[q][0]]
    return p1, p2


class PeerPullBroadcast:
    """Broadcast of the shared operand by peer-to-peer copies (DMA engines, no
    SMs), so the transfer does not compete with the persistent GEMM kernels the
    way a collective kernel does.  `views[r]` is rank r's buffer mapped into
    this process (torch symmetric memory); copies run on a private stream and
    one event per K-chunk tells the compute stream when its rows have landed.
    A one-element all-reduce on the same stream is the device-side barrier
    between the two phases of pull_plan()."""

    def __init__(self, torch, dist, views, src=0, group=None):
        self.torch, self.dist, self.views, self.src, self.group = torch, dist, views, src, group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.stream = torch.cuda.Stream()
        self.flag = torch.zeros(1, device=views[self.rank].device)

    def start(self, chunks):
        torch, dist = self.torch, self.dist
        mine = self.views[self.rank]
        self.stream.wait_stream(torch.cuda.current_stream())
        events = []
        with torch.cuda.stream(self.stream):
            # Nobody overwrites its buffer while a peer may still be reading it.
            dist.all_reduce(self.flag, group=self.group)
            for k0, k1 in chunks:
                p1, p2 = pull_plan(self.rank, self.world, self.src, k0, k1)
                for peer, r0, r1 in p1:
                    mine[r0:r1].copy_(self.views[peer][r0:r1], non_blocking=True)
                if self.world > 2:
                    dist.all_reduce(self.flag, group=self.group)
                for peer, r0, r1 in p2:
                    mine[r0:r1].copy_(self.views[peer][r0:r1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
                events.append(ev)
        return events


class PartitionedGemm:
    """C_p = alpha * A_p @ B + beta * C_p on every rank, B broadcast from `src`.

    `compute(alpha, A_chunk, B_chunk, beta, C)` must perform
    C = alpha*A_chunk@B_chunk + beta*C in place (the product path passes
    polygeist_b200.gemm, which enqueues on the current CUDA stream).
    """

    def __init__(self, dist, compute, src=0, chunk=1024, group=None, peer_broadcast=None,
                 first_chunk=0):
        self.dist = dist
        self.compute = compute
        self.src = src
        self.chunk = chunk
        self.first_chunk = first_chunk
        self.group = group
        self.peer_broadcast = peer_broadcast  # PeerPullBroadcast, or None for NCCL

    def run(self, alpha, A_p, B_local, beta, C_p):
        """`B_local`: the full [K,N] buffer on every rank; only `src`'s copy
        holds valid data on entry, all hold it on return."""
        dist = self.dist
        K = A_p.shape[1]
        chunks = k_chunks(K, self.chunk, self.first_chunk)
        world = dist.get_world_size(self.group)
        works = []
        if world > 1 and self.peer_broadcast is not None:
            pb = self.peer_broadcast
            events = pb.start(chunks)
            first = True
            for (k0, k1), ev in zip(chunks, events):
                pb.torch.cuda.current_stream().wait_event(ev)
                self.compute(alpha, A_p[:, k0:k1], B_local[k0:k1], beta if first else 1.0, C_p)
                first = False
            return C_p
        if world > 1:
            for k0, k1 in chunks:
                if k1 > k0:
                    works.append(dist.broadcast(B_local[k0:k1], src=self.src, group=self.group,
                                                async_op=True))
                else:
                    works.append(None)
        first = True
        for idx, (k0, k1) in enumerate(chunks):
            if world > 1 and works[idx] is not None:
                works[idx].wait()  # CUDA: orders the current stream after the transfer
            self.compute(alpha, A_p[:, k0:k1], B_local[k0:k1], beta if first else 1.0, C_p)
            first = False
        return C_p


class PartitionedSyrk:
    """Lower triangle of C = alpha*A@A^T + beta*C with the rows of C split over
    the ranks by equal triangular area.  Rank p owns rows [b[p], b[p+1]) of C
    and needs rows [0, b[p+1]) of A, which lives on `src`.

    A rank can only start once it holds its own rows of A, and with a row-wise
    broadcast the last rank receives those last.  The operand is therefore sent
    in K-slices: `src` packs the columns [k0,k1) of A into a contiguous
    [N, k1-k0] block, broadcasts it, and every rank accumulates
    C_p += alpha * A_p[:, k0:k1] @ A[0:r1, k0:k1]^T (beta applied with the first
    slice) while the next slice is in flight.

    `compute(alpha, A_rows_0_to_r1, beta, C_block, rows)` must update rows
    `rows=(r0,r1)` of the triangular result in place, `C_block` being those
    rows of C (the product path wraps pgb200SsyrkRows).
    """

    def __init__(self, dist, compute, src=0, kchunk=2048, group=None, align=128):
        self.dist = dist
        self.compute = compute
        self.src = src
        self.kchunk = kchunk
        self.group = group
        self.align = align
        self._packed = None
        self._packed_key = None

    def blocks(self, N):
        return syrk_row_blocks(N, self.dist.get_world_size(self.group), self.align)

    def run(self, alpha, A_local, beta, C_block):
        dist = self.dist
        N, K = A_local.shape
        world = dist.get_world_size(self.group)
        rank = dist.get_rank(self.group)
        b = self.blocks(N)
        r0, r1 = b[rank], b[rank + 1]
        if world == 1:
            self.compute(alpha, A_local, beta, C_block, (r0, r1))
            return C_block
        chunks = k_chunks(K, self.kchunk)
        key = (N, tuple(chunks), A_local.dtype, A_local.device)
        if self._packed is None or self._packed_key != key:
            # The packed K-slices are kept between calls of the same shape only.
            self._packed = [A_local.new_empty((N, k1 - k0)) for k0, k1 in chunks]
            self._packed_key = key
        works = []
        for (k0, k1), buf in zip(chunks, self._packed):
            if rank == self.src:
                buf.copy_(A_local[:, k0:k1])
            works.append(dist.broadcast(buf, src=self.src, group=self.group, async_op=True))
        first = True
        for w, buf in zip(works, self._packed):
            w.wait()
            if r1 > r0:
                self.compute(alpha, buf[:r1], beta if first else 1.0, C_block, (r0, r1))
            first = False
        return C_block
