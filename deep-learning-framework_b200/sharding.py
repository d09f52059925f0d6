"""Partition arithmetic of the multi-GPU configurations (one process per GPU).

Three partitions occur on the path, none of which needs a collective except the last:

* output blocks of the large NT GEMM: the ranks form a pr x pc grid, a rank holds one row-slab of X
  and one row-slab of W (= output columns) and writes its own block of Y.  The grid is the most
  square one, which minimises the operand bytes a rank reads and splits (M/pr + N/pc rows);
* batch items of the attention contractions;
* tokens of the Linear training step: Y and dX are row-sharded with W replicated, and the weight
  gradient dW = dY^T.X is a K-split whose full-size partials are summed with one all-reduce.

The reference's own multi-GPU mode slices the batch the same way (api_objects/vtensor.cpp:1034-1061)
but gathers and accumulates through cudaMemcpy on device 0 (api_objects/vmodule.cpp:855-863,
vtensor.cpp:443-451); here the exchange is torch.distributed (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations


def slab(n: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous [begin, end) share of n items for `rank`; the first n % world ranks get one more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def slabs(n: int, world: int) -> list[tuple[int, int]]:
    return [slab(n, world, r) for r in range(world)]


def grid2d(world: int, m: int, n: int) -> tuple[int, int]:
    """(pr, pc) with pr * pc == world that minimises the operand rows per rank, m / pr + n / pc."""
    if world < 1:
        raise ValueError(f"bad world size {world}")
    best = None
    for pr in range(1, world + 1):
        if world % pr:
            continue
        pc = world // pr
        cost = -(-m // pr) + -(-n // pc)
        if best is None or cost < best[0]:
            best = (cost, pr, pc)
    return best[1], best[2]


def block2d(m: int, n: int, world: int, rank: int) -> tuple[int, int, int, int]:
    """[m0, m1) x [n0, n1): the block of an m x n output that `rank` owns (row-major rank order)."""
    if not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    pr, pc = grid2d(world, m, n)
    m0, m1 = slab(m, pr, rank // pc)
    n0, n1 = slab(n, pc, rank % pc)
    return m0, m1, n0, n1


def linear_step_sharded(ops, x_local, w, b, dy_local, all_reduce):
    """One Linear training step on a token shard.

    ops: object with matmul(w, x) / add_bias(a, b) / matmul_backward_x(gy, w) /
    matmul_backward_w(gy, x, yvec, xvec) in the reference's semantics (the CPU oracle in tests, the
    GPU binding in production).  all_reduce(t) sums t over ranks in place and returns it.
    Returns (y_local, dx_local, dw_global).
    """
    yvec, xvec = w.shape
    y = ops.add_bias(ops.matmul(w, x_local), b)
    dx = ops.matmul_backward_x(dy_local, w)
    dw = all_reduce(ops.matmul_backward_w(dy_local, x_local, yvec, xvec))
    return y, dx, dw


def row_slabs(n: int, nslabs: int) -> list[tuple[int, int]]:
    """Non-empty contiguous [begin, end) row slabs of n rows, at most nslabs of them."""
    return [(a, b) for a, b in slabs(n, max(1, min(nslabs, n))) if b > a]


def linear_step_sharded_slabs(ops, x_local, w, b, dy_local, all_reduce_async, nslabs: int = 4):
    """The same step with the weight gradient computed and reduced in row slabs of dW.

    Slab s of dW needs columns [r0, r1) of dY only (dW[n, :] = sum_m dY[m, n] . X[m, :]), so its sum over
    ranks can start as soon as that slab's product is done and run under the products that follow (the
    later slabs, then Y and dX).  all_reduce_async(t) starts the in-place sum of t over ranks and returns
    an object with wait().  Every element is produced by the same loop and summed over the same ranks
    as in linear_step_sharded, so the result has the same bits.
    Returns (y_local, dx_local, dw_global).
    """
    import numpy as np

    yvec, xvec = w.shape
    dw = np.empty((yvec, xvec), np.float32)
    pending = []
    for r0, r1 in row_slabs(yvec, nslabs):
        dw[r0:r1] = ops.matmul_backward_w(np.ascontiguousarray(dy_local[:, r0:r1]), x_local, r1 - r0, xvec)
        pending.append(all_reduce_async(dw[r0:r1]))
    y = ops.add_bias(ops.matmul(w, x_local), b)
    dx = ops.matmul_backward_x(dy_local, w)
    for h in pending:
        h.wait()
    return y, dx, dw
