"""The device allocator behind VMath::mem_alloc / mem_free."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


def _stats(lib):
    a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
    assert lib.kai_mem_stats(0, C.byref(a), C.byref(b), C.byref(c)) == 0
    return a.value, b.value, c.value


def test_alignment_reuse_and_accounting(torch_cuda, pkg, vm):
    lib = pkg.load()
    live0, _, allocs0 = _stats(lib)
    ptrs = [vm.mem_alloc(0, s) for s in (1, 16, 100, 4096, 3 << 20)]
    assert all(p and p % 256 == 0 for p in ptrs)
    assert len(set(ptrs)) == len(ptrs)
    live1, _, allocs1 = _stats(lib)
    assert live1 - live0 >= 1 + 16 + 100 + 4096 + (3 << 20) and allocs1 - allocs0 <= 5
    for p in ptrs:
        vm.mem_free(0, p)
    live2, cached2, allocs2 = _stats(lib)
    assert live2 == live0 and cached2 >= live1 - live0
    again = vm.mem_alloc(0, 3 << 20)         # same size class: served from the cache, no driver call
    assert again == ptrs[-1] and _stats(lib)[2] == allocs2
    torch_cuda.cuda.synchronize()
    vm.mem_free(0, again)
    assert lib.kai_mem_trim(0) == 0 and _stats(lib)[1] == 0


def test_pitched_rows_are_tma_aligned(torch_cuda, pkg):
    lib = pkg.load()
    p, pitch = C.c_void_p(), C.c_int64()
    assert lib.kai_mem_alloc_pitched(0, 128, 10 * 4, C.byref(p), C.byref(pitch)) == 0   # N = 10 floats per row
    assert pitch.value % 128 == 0 and pitch.value >= 40 and p.value % 256 == 0
    assert lib.kai_mem_free(0, p) == 0


def test_errors(torch_cuda, pkg, vm):
    lib = pkg.load()
    with pytest.raises(pkg.KaiError):
        vm.mem_free(0, 0xdead0000)           # not ours
    vm.mem_free(0, 0)                        # freeing NULL is a no-op, like free()
    out = C.c_void_p()
    assert lib.kai_mem_alloc(0, -5, C.byref(out)) == pkg.capi.E_INVALID_ARG
    assert lib.kai_mem_alloc(-1, 64, C.byref(out)) == pkg.capi.E_NO_HOST_PATH


def test_memory_from_the_allocator_feeds_the_gemm(torch_cuda, vm, port):
    import numpy as np
    torch = torch_cuda
    M, N, K = 64, 96, 128
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((M, K), dtype=np.float32), rng.standard_normal((N, K), dtype=np.float32)
    pa, pb, pc = (vm.mem_alloc(0, n * 4) for n in (M * K, N * K, M * N))
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    assert rt.cudaMemcpy(pa, a.ctypes.data, a.nbytes, 1) == 0
    assert rt.cudaMemcpy(pb, b.ctypes.data, b.nbytes, 1) == 0
    vm.sgemm(0, 0, pc, pa, pb, M, N, K, path=2)
    out = np.empty((M, N), np.float32)
    assert rt.cudaMemcpy(out.ctypes.data, pc, out.nbytes, 2) == 0
    np.testing.assert_allclose(out, port.matmul(b, a), rtol=1e-4, atol=1e-4)
    for p in (pa, pb, pc):
        vm.mem_free(0, p)
