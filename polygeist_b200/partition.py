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


def k_chunks(K, chunk):
    chunk = max(1, int(chunk))
    return [(k0, min(K, k0 + chunk)) for k0 in range(0, K, chunk)] or [(0, 0)]


class PartitionedGemm:
    """C_p = alpha * A_p @ B + beta * C_p on every rank, B broadcast from `src`.

    `compute(alpha, A_chunk, B_chunk, beta, C)` must perform
    C = alpha*A_chunk@B_chunk + beta*C in place (the product path passes
    polygeist_b200.gemm, which enqueues on the current CUDA stream).
    """

    def __init__(self, dist, compute, src=0, chunk=1024, group=None):
        self.dist = dist
        self.compute = compute
        self.src = src
        self.chunk = chunk
        self.group = group

    def run(self, alpha, A_p, B_local, beta, C_p):
        """`B_local`: the full [K,N] buffer on every rank; only `src`'s copy
        holds valid data on entry, all hold it on return."""
        dist = self.dist
        K = A_p.shape[1]
        chunks = k_chunks(K, self.chunk)
        world = dist.get_world_size(self.group)
        works = []
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
