"""world_size-2 gloo test of the partition arithmetic: the sharded Linear step (token-split Y/dX,
K-split dW + all-reduce) and the column-sharded GEMM reproduce the unsharded oracle result."""
import importlib
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_slab_covers_everything():
    sh = importlib.import_module("deep-learning-framework_b200.sharding")
    for n in (0, 1, 7, 8, 8192, 1000003):
        for world in (1, 2, 3, 4, 8):
            parts = sh.slabs(n, world)
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in parts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sh.slab(4, 2, 2)


def test_block2d_tiles_the_output():
    sh = importlib.import_module("deep-learning-framework_b200.sharding")
    assert sh.grid2d(1, 8192, 8192) == (1, 1)
    assert sh.grid2d(4, 8192, 8192) == (2, 2)
    assert sorted(sh.grid2d(8, 8192, 8192)) == [2, 4]
    assert sh.grid2d(8, 16, 8192) == (1, 8)          # a skinny output splits along its long side only
    for m, n in ((8192, 8192), (50, 40), (7, 3), (1, 9)):
        for world in (1, 2, 3, 4, 6, 8):
            cover = np.zeros((m, n), np.int32)
            for r in range(world):
                m0, m1, n0, n1 = sh.block2d(m, n, world, r)
                cover[m0:m1, n0:n1] += 1
            assert (cover == 1).all(), (m, n, world)
    with pytest.raises(ValueError):
        sh.block2d(4, 4, 2, 2)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    import oracle
    sh = importlib.import_module("deep-learning-framework_b200.sharding")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = oracle.Oracle("port")
    rng = np.random.default_rng(7)  # every rank draws the same global tensors
    tokens, d_in, d_out = 50, 24, 40
    x = rng.standard_normal((tokens, d_in), dtype=np.float32)
    w = rng.standard_normal((d_out, d_in), dtype=np.float32)
    b = rng.standard_normal(d_out, dtype=np.float32)
    dy = rng.standard_normal((tokens, d_out), dtype=np.float32)
    t0, t1 = sh.slab(tokens, world, rank)

    def all_reduce(a):
        t = torch.from_numpy(a)
        dist.all_reduce(t)
        return a

    y, dx, dw = sh.linear_step_sharded(orc, np.ascontiguousarray(x[t0:t1]), w, b, np.ascontiguousarray(dy[t0:t1]),
                                       all_reduce)
    # the same step with dW computed and reduced in row slabs (each slab's reduce overlaps the next products)
    def all_reduce_async(a):
        return dist.all_reduce(torch.from_numpy(a), async_op=True)

    y_s, dx_s, dw_s = sh.linear_step_sharded_slabs(orc, np.ascontiguousarray(x[t0:t1]), w, b,
                                                   np.ascontiguousarray(dy[t0:t1]), all_reduce_async, nslabs=3)
    assert np.array_equal(y_s, y) and np.array_equal(dx_s, dx)
    # column-sharded GEMM: rank owns W rows n0:n1 = output columns n0:n1
    n0, n1 = sh.slab(d_out, world, rank)
    y_cols = orc.matmul(np.ascontiguousarray(w[n0:n1]), x)
    # block-sharded GEMM: rank owns X rows m0:m1 and W rows c0:c1
    m0, m1, c0, c1 = sh.block2d(tokens, d_out, world, rank)
    y_block = orc.matmul(np.ascontiguousarray(w[c0:c1]), np.ascontiguousarray(x[m0:m1]))
    np.savez(Path(tmp) / f"rank{rank}.npz", y=y, dx=dx, dw=dw, dw_slabs=dw_s, y_cols=y_cols, t=np.array([t0, t1]),
             n=np.array([n0, n1]), y_block=y_block, blk=np.array([m0, m1, c0, c1]))
    dist.destroy_process_group()


def test_sharded_linear_step_matches_unsharded(tmp_path):
    import torch.multiprocessing as mp

    import oracle
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    orc = oracle.Oracle("port")
    rng = np.random.default_rng(7)
    tokens, d_in, d_out = 50, 24, 40
    x = rng.standard_normal((tokens, d_in), dtype=np.float32)
    w = rng.standard_normal((d_out, d_in), dtype=np.float32)
    b = rng.standard_normal(d_out, dtype=np.float32)
    dy = rng.standard_normal((tokens, d_out), dtype=np.float32)
    y_full = orc.add_bias(orc.matmul(w, x), b)
    dx_full = orc.matmul_backward_x(dy, w)
    dw_full = orc.matmul_backward_w(dy, x, d_out, d_in)
    y_plain = orc.matmul(w, x)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    # row-sharded outputs are bit-identical: each row is computed by the same loop
    np.testing.assert_array_equal(np.concatenate([p["y"] for p in parts]), y_full)
    np.testing.assert_array_equal(np.concatenate([p["dx"] for p in parts]), dx_full)
    np.testing.assert_array_equal(np.concatenate([p["y_cols"] for p in parts], axis=1), y_plain)
    y_blocks = np.full_like(y_plain, np.nan)
    for p in parts:
        m0, m1, c0, c1 = p["blk"]
        y_blocks[m0:m1, c0:c1] = p["y_block"]
    np.testing.assert_array_equal(y_blocks, y_plain)
    # the K-split gradient changes the summation order: equal up to fp32 rounding, same on all ranks
    np.testing.assert_allclose(parts[0]["dw"], dw_full, rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(parts[0]["dw"], parts[1]["dw"])
    # slab-wise reduction: bit-equal to the whole-tensor form
    for p in parts:
        np.testing.assert_array_equal(p["dw_slabs"], p["dw"])
