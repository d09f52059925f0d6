"""The recurrent layers' call pattern (api_objects/vtensor.cpp:2456-2495): per timestep one matmul of the previous
state (acc = false) and one of the input (acc = true) into the same interior slice of a [ntimes, ndat, gates]
tensor.  Checked against the CPU restatement, and against the batched form in which the input products of all
timesteps are one GEMM and only the recurrent product stays in the loop."""
import numpy as np
import pytest

from helpers import rel_fro, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dims", [(6, 5, 24, 16, 1), (8, 32, 96, 64, 4), (4, 64, 512, 256, 4)])
def test_timestep_matmuls_on_interior_pointers(torch_cuda, vm, port, dims):
    torch = torch_cuda
    ntimes, ndat, ninp, nrec, ngates = dims
    G = ngates * nrec
    rng = np.random.default_rng(ntimes * 1000 + ndat)
    x = rng.standard_normal((ntimes, ndat, ninp)).astype(np.float32)
    wi = (rng.standard_normal((G, ninp)) / np.sqrt(ninp)).astype(np.float32)
    wr = (rng.standard_normal((G, nrec)) / np.sqrt(nrec)).astype(np.float32)
    b = rng.standard_normal(G).astype(np.float32)

    # CPU: the reference's order.  The state fed back is the first gate's slice through tanh (a stand-in for
    # the cell update, which is not a contraction).
    aff = np.zeros((ntimes, ndat, G), np.float32)
    rec = np.zeros((ntimes, ndat, nrec), np.float32)
    for t in range(ntimes):
        if t > 0:
            port.matmul_into(aff[t], wr, rec[t - 1], G, ndat, nrec, acc=False)
        port.matmul_into(aff[t], wi, x[t], G, ndat, ninp, acc=True)
        aff[t] = port.add_bias(aff[t], b)
        rec[t] = port.activate(np.ascontiguousarray(aff[t][:, :nrec]), 4)

    dx, dwi, dwr, db = (to_dev(torch, v) for v in (x, wi, wr, b))

    def run(batched):
        daff = torch.zeros((ntimes, ndat, G), device="cuda")
        drec = torch.zeros((ntimes, ndat, nrec), device="cuda")
        gate0 = torch.empty((ndat, nrec), device="cuda")
        if batched:   # all input products at once: [ntimes * ndat, ninp] . wi^T
            vm.matmul(0, daff, dwi, dx, G, ntimes * ndat, ninp, False)
        for t in range(ntimes):
            if batched:
                if t > 0:
                    vm.matmul(0, daff[t], dwr, drec[t - 1], G, ndat, nrec, True)
            else:
                if t > 0:
                    vm.matmul(0, daff[t], dwr, drec[t - 1], G, ndat, nrec, False)
                vm.matmul(0, daff[t], dwi, dx[t], G, ndat, ninp, True)
            vm.add_bias(0, daff[t], daff[t], db, ndat, G)
            gate0.copy_(daff[t][:, :nrec])
            vm.activate(0, drec[t], gate0, ndat, nrec, 4, None)
        torch.cuda.synchronize()
        return to_host(daff), to_host(drec)

    for batched in (False, True):
        got_aff, got_rec = run(batched)
        assert rel_fro(got_aff, aff) < 2e-5 * np.sqrt(ntimes), f"batched={batched}"
        assert rel_fro(got_rec, rec) < 2e-5 * np.sqrt(ntimes), f"batched={batched}"


@pytest.mark.parametrize("layout", [0, 1, 2])
@pytest.mark.parametrize("count", [1, 5, 40])
def test_grouped_products_match_single_calls(torch_cuda, vm, port, layout, count):
    """kai_sgemm_grouped: `count` products of one shape in one launch (more than 32 groups take two)."""
    torch = torch_cuda
    M, N, K = 48, 80, 72
    rng = np.random.default_rng(count * 10 + layout)
    sa = (M, K) if layout != 2 else (K, M)
    sb = (N, K) if layout == 0 else (K, N)
    a = rng.standard_normal((count,) + sa).astype(np.float32)
    b = rng.standard_normal((count,) + sb).astype(np.float32)
    da, db = to_dev(torch, a), to_dev(torch, b)
    c = torch.ones((count, M, N), device="cuda")
    want = torch.ones((count, M, N), device="cuda")
    vm.sgemm_grouped(0, layout, [c[i] for i in range(count)], [da[i] for i in range(count)],
                     [db[i] for i in range(count)], M, N, K, accumulate=True)
    for i in range(count):
        vm.sgemm(0, layout, want[i], da[i], db[i], M, N, K, accumulate=True, path=2)
    torch.cuda.synchronize()
    # single calls of this size split the reduction over a cluster, the grouped launch does not: same values up
    # to the order of the fp32 sums
    assert float((c - want).abs().max()) <= 2e-5 * float(want.abs().max())
    ref = {0: lambda i: a[i] @ b[i].T, 1: lambda i: a[i] @ b[i], 2: lambda i: a[i].T @ b[i]}[layout]
    np.testing.assert_allclose(to_host(c[count - 1]), 1.0 + ref(count - 1), rtol=1e-4, atol=1e-4)


def test_grouped_input_products_of_a_recurrent_layer(torch_cuda, vm, port):
    """The per-timestep input products (acc = true into interior slices of one tensor) as ONE grouped launch,
    with the shared weight as every group's B operand."""
    torch = torch_cuda
    ntimes, ndat, ninp, G = 12, 16, 40, 96
    rng = np.random.default_rng(3)
    x = rng.standard_normal((ntimes, ndat, ninp)).astype(np.float32)
    wi = rng.standard_normal((G, ninp)).astype(np.float32)
    aff0 = rng.standard_normal((ntimes, ndat, G)).astype(np.float32)
    want = aff0.copy()
    for t in range(ntimes):
        port.matmul_into(want[t], wi, x[t], G, ndat, ninp, acc=True)
    dx, dwi, daff = to_dev(torch, x), to_dev(torch, wi), to_dev(torch, aff0)
    vm.sgemm_grouped(0, 0, [daff[t] for t in range(ntimes)], [dx[t] for t in range(ntimes)], [dwi] * ntimes,
                     ndat, G, ninp, accumulate=True)
    torch.cuda.synchronize()
    np.testing.assert_allclose(to_host(daff), want, rtol=2e-5, atol=2e-5)
