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


def slice_groups(nslices, grow=True):
    """Groups of consecutive K-slices that are multiplied by one product each:
    [first, last) index pairs of sizes 1, 1, 2, 4, 8, ... (the last one takes
    what is left).  The slices travel one by one, so the first product starts
    as soon as one slice has landed; a product of few long-K calls is faster
    than one of many short ones (fp32 32768^3 on one GPU: 16 slices of 2048
    cost 9 % over the unsliced product, 4 of 8192 cost 3 %), and the transfer
    is several times faster than the product, so the later, longer groups
    have landed long before they are needed.  grow=False: one slice per group."""
    if not grow:
        return [(i, i + 1) for i in range(nslices)]
    groups, start, size = [], 0, 1
    while start < nslices:
        end = min(nslices, start + size)
        groups.append((start, end))
        if len(groups) >= 2:
            size *= 2
        start = end
    return groups


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


def pull_schedule(rank, world, src, chunks):
    """The copy-engine broadcast of all K-slices as one ordered list of
    operations for `rank`'s copy stream:

      ("pull", peer, r0, r1)  copy rows [r0,r1) from `peer`'s buffer into mine
      ("signal", c)           tell the other non-source ranks that my piece of
                              slice c has landed (after the phase-1 pull; the
                              source has no piece and skips it)
      ("wait", peer, c)       wait until `peer` has signalled slice c (before
                              pulling its piece)
      ("ready", c)            slice c is complete here: record its event

    No rank ever waits for something that comes later in the signaller's own
    list than an operation that waits for this rank, so the lists cannot
    deadlock (checked by simulation in the tests)."""
    ops = []
    for c, (k0, k1) in enumerate(chunks):
        p1, p2 = pull_plan(rank, world, src, k0, k1)
        for peer, r0, r1 in p1:
            ops.append(("pull", peer, r0, r1))
        if world > 2:
            ops.append(("signal", c))     # the source has nothing to signal: phase boundary only
        for peer, r0, r1 in p2:
            ops.append(("wait", peer, c))
            ops.append(("pull", peer, r0, r1))
        ops.append(("ready", c))
    return ops


def stream_memops():
    """(write_value, wait_value): 32-bit stream memory operations of the CUDA
    driver through cuda-python.  write_value(stream, ptr, v) stores v at ptr in
    stream order; wait_value(stream, ptr, v) holds the stream until the word at
    ptr is >= v.  Neither launches a kernel, so they make progress while
    persistent kernels hold every SM."""
    from cuda.bindings import driver

    def check(ret, what):
        err = ret[0] if isinstance(ret, tuple) else ret
        if err != driver.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"{what} failed with {err}")

    geq = int(driver.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_GEQ)

    def write_value(stream, ptr, value):
        check(driver.cuStreamWriteValue32(driver.CUstream(stream), driver.CUdeviceptr(ptr),
                                          int(value), 0), "cuStreamWriteValue32")

    def wait_value(stream, ptr, value):
        check(driver.cuStreamWaitValue32(driver.CUstream(stream), driver.CUdeviceptr(ptr),
                                         int(value), geq), "cuStreamWaitValue32")

    return write_value, wait_value


class PeerPullBroadcast:
    """Broadcast of the shared operand by peer-to-peer copies (DMA engines, no
    SMs), so the transfer does not compete with the persistent GEMM kernels the
    way a collective kernel does: those kernels fill the register file of every
    SM, a collective's CTAs only run between two of them, and the broadcast ends
    up in series with the products (measured at 2 GPUs, fp32 32768^3: 160 ms per
    step with the NCCL broadcast against 139 ms for the products alone).

    `views[r]` is rank r's buffer mapped into this process (torch symmetric
    memory); copies run on a private stream and one event per K-slice tells the
    compute stream when its rows have landed.  One small all-reduce per call on
    that stream (it runs before the first product, when the GPU is idle) keeps
    any rank from overwriting rows a peer may still be reading.

    Between the two phases of pull_plan() a rank must know that the owner of a
    piece has received it.  With `flags` (flags[r] = rank r's int32 [world,
    slots] array, mapped like `views`) and `memops` (see stream_memops) this is
    a word per (owner, slice) that the owner sets to the call number in every
    peer's array after its phase-1 copy - a 4-byte copy in stream order (the
    driver refuses a stream memory operation that writes a peer-mapped word:
    CUDA_ERROR_INVALID_VALUE) - and that the peer's copy stream waits for with
    a stream memory operation on its own memory: no kernel at all.  Without them an all-reduce per slice is the barrier (its
    kernel waits for the running product)."""

    def __init__(self, torch, dist, views, src=0, group=None, flags=None, memops=None):
        self.torch, self.dist, self.views, self.src, self.group = torch, dist, views, src, group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.stream = torch.cuda.Stream()
        self.flag = torch.zeros(1, device=views[self.rank].device)
        self.flags = flags
        self.memops = memops if flags is not None else None
        self.call = 0
        self._numbers = None          # device words 1, 2, 3, ...: sources of the signal copies
        self._numbers_base = 0

    def _number(self, value):
        """A one-element device tensor holding `value` (a call number)."""
        torch = self.torch
        if self._numbers is None or not (self._numbers_base <= value < self._numbers_base + 4096):
            self._numbers_base = value
            self._numbers = torch.arange(value, value + 4096, dtype=torch.int32,
                                         device=self.views[self.rank].device)
        i = value - self._numbers_base
        return self._numbers[i:i + 1]

    def start(self, chunks):
        torch, dist = self.torch, self.dist
        mine = self.views[self.rank]
        signalled = self.flags is not None and self.world > 2
        if signalled and len(chunks) > self.flags[self.rank].shape[1]:
            raise ValueError("more K-slices than signal slots")
        self.call += 1
        number = self._number(self.call) if signalled else None
        self.stream.wait_stream(torch.cuda.current_stream())
        events = []
        with torch.cuda.stream(self.stream):
            # Nobody overwrites its buffer while a peer may still be reading it.
            dist.all_reduce(self.flag, group=self.group)
            handle = self.stream.cuda_stream
            for op in pull_schedule(self.rank, self.world, self.src, chunks):
                if op[0] == "pull":
                    _, peer, r0, r1 = op
                    mine[r0:r1].copy_(self.views[peer][r0:r1], non_blocking=True)
                elif op[0] == "signal":
                    if not signalled:
                        dist.all_reduce(self.flag, group=self.group)
                    elif self.rank != self.src:
                        for q in range(self.world):
                            if q == self.rank or q == self.src:
                                continue
                            self.flags[q][self.rank, op[1]:op[1] + 1].copy_(number, non_blocking=True)
                elif op[0] == "wait":
                    if signalled:
                        word = self.flags[self.rank][op[1], op[2]:op[2] + 1]
                        self.memops[1](handle, word.data_ptr(), self.call)
                else:
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
                 first_chunk=0, grow=True):
        self.dist = dist
        self.compute = compute
        self.src = src
        self.chunk = chunk
        self.first_chunk = first_chunk
        self.grow = grow                      # slice_groups(): longer products as the run goes on
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
            for g0, g1 in slice_groups(len(chunks), self.grow):
                pb.torch.cuda.current_stream().wait_event(events[g1 - 1])  # slices land in order
                k0, k1 = chunks[g0][0], chunks[g1 - 1][1]
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
        for g0, g1 in slice_groups(len(chunks), self.grow and world > 1):
            if world > 1:
                for idx in range(g0, g1):
                    if works[idx] is not None:
                        works[idx].wait()  # CUDA: orders the current stream after the transfer
            k0, k1 = chunks[g0][0], chunks[g1 - 1][1]
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
